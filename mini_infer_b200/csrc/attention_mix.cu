// Attention whose heads are not independent: after the scaled dot products every head's score of a
// (query, key) pair is soft-capped, score <- cap * tanh(score / cap), and then replaced by a mix of all
// heads' scores of that pair, score_h <- sum_g mix[h, g] * score_g, before the softmax over the visible
// keys.  A block therefore owns ALL heads of its queries.  Keys and values may have different sizes per
// head, so the two caches have their own row lengths:
//
//   k_cache [page, kv_head, page_size, dk]      v_cache [page, kv_head, page_size, dv]
//
// Masking is positional: key j is visible from the query at absolute position p iff j <= p and
// (window == 0 or j > p - window or j < keep_first): behind a window the first keep_first keys of a request
// stay visible, at their true positions.  A value row may lie inside a longer row of memory (`vrs`, the
// distance between two tokens' value rows in elements): values that are the leading part of their keys are
// read from the key cache itself.  Key tiles are aligned to absolute positions and every sum runs in an
// order that depends on the model's sizes only, so the result does not depend on how a prompt was cut.
//
// rope_store: optionally each query and key head divided by its root mean square and multiplied by a gain
// per dimension (shared by the heads), then rotary encoding of the first rot_dim dimensions of every query
// and key head (dimension i is paired with i + rot_dim/2, or, `neighbours`, dimension 2i with 2i + 1), cache
// write of keys and values.  With `v_first` a token's values are first blended with another layer's values of
// the same token, v <- (1 - lam) v + lam v_first (float rows of their own stride; lam one float on the device).
//
// `sink`: the softmax counts one key more, of score 0 and without a value: p_j = exp(s_j) / (1 + sum exp(s_j)).
// The running maximum then starts at 0 and the running sum at 1 instead of at -inf and 0.
//
// `head_bias` (a number per head): no softmax.  The weight of a visible key is logistic(score + head_bias[h]) by
// itself, and a query's weights are not normalised over its keys: out = sum_j logistic(s_j + b_h) v_j.

#include "common.cuh"

namespace mi {

// one block per token; qkv row: [nh*dk | nkv*dk | nkv*dv] float
template <typename AT>
__global__ void __launch_bounds__(256)
rope_store_kernel(const float* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                  const int* __restrict__ slot_mapping, AT* __restrict__ q_out, AT* __restrict__ k_cache,
                  AT* __restrict__ v_cache, int nh, int nkv, int dk, int dv, int rot_dim, int page_size,
                  const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps, int neighbours,
                  const float* __restrict__ v_first, int64_t v_first_stride, const float* __restrict__ lam_ptr) {
    extern __shared__ float trig[];                 // cos and sin of this token's rot_dim / 2 angles
    float* inv_rms = trig + (rot_dim > 0 ? rot_dim : 1);    // [nh + nkv], with head norms only
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    const float* row = qkv + (int64_t)t * ((int64_t)(nh + nkv) * dk + (int64_t)nkv * dv);
    const float pos = (float)positions[t];
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const int half = rot_dim / 2;
    const int nqk = (nh + nkv) * dk;
    // the angles depend on the position and the pair only: once per token, not once per head
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = pos * inv_freq[i];
        trig[i] = cosf(ang);
        trig[half + i] = sinf(ang);
    }
    const bool normed = q_gain != nullptr;
    if (normed) {
        // a warp per head; a lane adds its dimensions in ascending order, then the lanes are added: an order
        // that depends on dk only
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
        for (int head = warp; head < nh + nkv; head += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < dk; c += 32) { const float x = row[head * dk + c]; ss += x * x; }
            ss = warp_sum(ss);
            if (lane == 0) inv_rms[head] = 1.0f / sqrtf(ss / (float)dk + eps);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nqk; idx += blockDim.x) {
        const int head = idx / dk, c = idx - head * dk;
        float v = row[idx];
        const float* gain = head < nh ? q_gain : k_gain;
        if (normed) v = v * inv_rms[head] * gain[c];
        if (c < rot_dim) {
            // the first of a pair becomes u cos - v sin, the second v cos + u sin
            const bool first = neighbours ? !(c & 1) : c < half;
            const int i = neighbours ? c >> 1 : (c < half ? c : c - half);
            const float cs = trig[i], sn = trig[half + i];
            const int co = neighbours ? (c ^ 1) : (c < half ? c + half : c - half);
            float other = row[head * dk + co];
            if (normed) other = other * inv_rms[head] * gain[co];
            v = first ? v * cs - other * sn : v * cs + other * sn;
        }
        if (head < nh) {
            q_out[(int64_t)t * nh * dk + idx] = from_float<AT>(v);
        } else if (slot >= 0) {
            const int hk = head - nh;
            const int page = slot / page_size, off = slot - page * page_size;
            k_cache[(((int64_t)page * nkv + hk) * page_size + off) * dk + c] = from_float<AT>(v);
        }
    }
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        const float lam = v_first ? lam_ptr[0] : 0.f;
        for (int idx = threadIdx.x; idx < nkv * dv; idx += blockDim.x) {
            const int hk = idx / dv, c = idx - hk * dv;
            float v = row[nqk + idx];
            if (v_first) v = (1.0f - lam) * v + lam * v_first[(int64_t)t * v_first_stride + idx];
            v_cache[(((int64_t)page * nkv + hk) * page_size + off) * dv + c] = from_float<AT>(v);
        }
    }
}

// Head sizes and the rotated part multiples of four (of eight where halves are paired), rows on 16-byte
// boundaries: a warp per query, key or value head, grid (tokens, ceil((nh + 2 nkv) / 8)).  A lane keeps its
// groups of four of the head in registers from the sum of squares to the store (heads of up to 128 CH).  The
// squares are added per lane in ascending order and then over the lanes: an order that depends on dk only.
template <typename AT, int CH>
__global__ void __launch_bounds__(256)
rope_store_vec_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                      const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping, AT* __restrict__ q_out,
                      AT* __restrict__ k_cache, AT* __restrict__ v_cache, int nh, int nkv, int dk, int dv, int rot_dim,
                      int page_size, const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                      int neighbours, const float* __restrict__ v_first, int64_t v_first_stride,
                      const float* __restrict__ lam_ptr) {
    extern __shared__ float trig[];                 // cos and sin of this token's rot_dim / 2 angles
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * 8 + warp;
    const int half = rot_dim / 2;
    const int nqk = (nh + nkv) * dk;
    const float* row = qkv + (int64_t)t * ((int64_t)nqk + (int64_t)nkv * dv);
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if ((int)blockIdx.y * 8 < nh + nkv) {           // a block of value heads alone needs no angles
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float ang = pos * inv_freq[i];
            trig[i] = cosf(ang);
            trig[half + i] = sinf(ang);
        }
    }
    __syncthreads();
    if (head >= nh + 2 * nkv) return;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot - page * page_size;
    if (head >= nh + nkv) {
        if (slot < 0) return;
        const int hk = head - nh - nkv;
        const float4* src = reinterpret_cast<const float4*>(row + nqk + hk * dv);
        const float4* fst = v_first ? reinterpret_cast<const float4*>(v_first + (int64_t)t * v_first_stride + hk * dv)
                                    : nullptr;
        const float lam = v_first ? lam_ptr[0] : 0.f;
        AT* dst = v_cache + (((int64_t)page * nkv + hk) * page_size + off) * dv;
        for (int c = lane; c < (dv >> 2); c += 32) {
            float4 v = src[c];
            if (fst) {
                const float4 f = fst[c];
                v.x = (1.0f - lam) * v.x + lam * f.x;
                v.y = (1.0f - lam) * v.y + lam * f.y;
                v.z = (1.0f - lam) * v.z + lam * f.z;
                v.w = (1.0f - lam) * v.w + lam * f.w;
            }
            store4(dst + 4 * c, v);
        }
        return;
    }
    const bool is_q = head < nh;
    if (!is_q && slot < 0) return;
    const float4* hrow = reinterpret_cast<const float4*>(row + head * dk);
    const int nc = dk >> 2;
    float4 x[CH];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = lane + 32 * j;
        x[j] = c < nc ? hrow[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += x[j].x * x[j].x;
        ss += x[j].y * x[j].y;
        ss += x[j].z * x[j].z;
        ss += x[j].w * x[j].w;
    }
    const bool normed = q_gain != nullptr;
    const float4* gain = reinterpret_cast<const float4*>(is_q ? q_gain : k_gain);
    float r = 1.0f;
    if (normed) {
        ss = warp_sum(ss);
        r = 1.0f / sqrtf(ss / (float)dk + eps);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = lane + 32 * j;
            if (c < nc) {
                const float4 g = gain[c];
                x[j].x = x[j].x * r * g.x;
                x[j].y = x[j].y * r * g.y;
                x[j].z = x[j].z * r * g.z;
                x[j].w = x[j].w * r * g.w;
            }
        }
    }
    AT* dst = is_q ? q_out + (int64_t)t * nh * dk + head * dk
                   : k_cache + (((int64_t)page * nkv + (head - nh)) * page_size + off) * dk;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = lane + 32 * j;
        if (c >= nc) continue;
        float4 v = x[j];
        if (4 * c < rot_dim) {
            if (neighbours) {
                // (x, y) is pair 2c, (z, w) pair 2c + 1: the first becomes u cos - v sin, the second v cos + u sin
                const float c0 = trig[2 * c], s0 = trig[half + 2 * c];
                const float c1 = trig[2 * c + 1], s1 = trig[half + 2 * c + 1];
                v.x = x[j].x * c0 - x[j].y * s0;
                v.y = x[j].y * c0 + x[j].x * s0;
                v.z = x[j].z * c1 - x[j].w * s1;
                v.w = x[j].w * c1 + x[j].z * s1;
            } else {
                // dimension i < half is paired with i + half: the partner group lies with another lane
                const bool first = 4 * c < half;
                const int pc = first ? c + (half >> 2) : c - (half >> 2);
                float4 o = hrow[pc];
                if (normed) {
                    const float4 g = gain[pc];
                    o.x = o.x * r * g.x;
                    o.y = o.y * r * g.y;
                    o.z = o.z * r * g.z;
                    o.w = o.w * r * g.w;
                }
                const int i = 4 * (first ? c : pc);
                const float sg = first ? -1.0f : 1.0f;
                v.x = x[j].x * trig[i] + sg * (o.x * trig[half + i]);
                v.y = x[j].y * trig[i + 1] + sg * (o.y * trig[half + i + 1]);
                v.z = x[j].z * trig[i + 2] + sg * (o.z * trig[half + i + 2]);
                v.w = x[j].w * trig[i + 3] + sg * (o.w * trig[half + i + 3]);
            }
        }
        store4(dst + 4 * c, v);
    }
}

// ---------------------------------------------------------------------------
// Block = 256 threads, QT consecutive queries of one request with all H heads: R = H * QT rows, row
// r = h * QT + i.  Warp w owns the rows [w * rpw, (w + 1) * rpw) through softmax and P.V; lane l owns the
// value columns l, l + 32, ...  Per key tile of KT keys: raw scores of all rows into shared memory, cap,
// mix over heads (into a second buffer), mask, running softmax per row, P.V.
// ---------------------------------------------------------------------------
template <typename AT, int CPL>     // CPL = ceil(dv / 32) value columns per lane
struct MixCfg {
    static constexpr int RPW = CPL >= 8 ? 8 : 16;       // most rows per warp
};

template <typename AT, int CPL>
__global__ void __launch_bounds__(256)
attn_mix_kernel(const AT* __restrict__ q, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache,
                const float* __restrict__ mix, const int* __restrict__ block_table, const int* __restrict__ q_start,
                const int* __restrict__ kv_len, AT* __restrict__ out, int H, int G, int dk, int dv, int page_size,
                int max_pages, int window, float scale, float cap, int QT, int KT, int rpw, int keep_first, int vrs,
                int sink, const float* __restrict__ head_bias) {
    constexpr int RPW = MixCfg<AT, CPL>::RPW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    wait_for_earlier_kernels();
    const int b = blockIdx.y, qt = blockIdx.x;
    const int q0 = q_start[b], q_len = q_start[b + 1] - q0;
    if (qt * QT >= q_len) return;
    const int kvl = kv_len[b];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = H * QT;
    const int rep = H / G;
    const int ksd = dk + (sizeof(AT) == 2 ? 2 : 1);     // row stride of a key in shared memory: odd in words
    const int kv_elems = G * KT * (ksd > dv ? ksd : dv);
    const int SP = KT + 1;
    float* S1 = reinterpret_cast<float*>(smem_raw);             // [R][KT+1] capped scores
    float* S2 = S1 + R * SP;                                     // [R][KT+1] mixed scores, then P
    float* Mx = S2 + R * SP;                                     // [H*H]
    int* slot_of = reinterpret_cast<int*>(Mx + H * H);           // [KT] page * page_size + offset, or -1
    AT* Qs = reinterpret_cast<AT*>(slot_of + KT);                // [R][dk]
    AT* KV = Qs + (int64_t)R * dk;                               // keys [G][KT][ksd], then values [G][KT][dv]
    (void)kv_elems;

    const int nq = min(QT, q_len - qt * QT);
    const int p_lo = kvl - q_len + qt * QT;                      // absolute position of local query 0
    const int p_hi = p_lo + nq - 1;

    for (int idx = tid; idx < R * dk; idx += 256) {
        const int r = idx / dk, c = idx - r * dk;
        const int h = r / QT, i = r - h * QT;
        AT v = from_float<AT>(0.f);
        if (i < nq) v = q[((int64_t)(q0 + qt * QT + i) * H + h) * dk + c];
        Qs[idx] = v;
    }
    if (mix) for (int idx = tid; idx < H * H; idx += 256) Mx[idx] = mix[idx];

    float m_run[RPW], l_run[RPW], acc[RPW][CPL];
    int g_of[RPW];
#pragma unroll
    for (int m = 0; m < RPW; ++m) {
        m_run[m] = sink ? 0.f : -INFINITY; l_run[m] = sink ? 1.f : 0.f;
        const int r = warp * rpw + m;
        g_of[m] = (r < R ? r / QT : 0) / rep;
#pragma unroll
        for (int n = 0; n < CPL; ++n) acc[m][n] = 0.f;
    }

    int k_begin = 0;
    if (window > 0) k_begin = max(0, p_lo - window + 1);
    k_begin = (k_begin / KT) * KT;
    const int k_end = min(kvl, p_hi + 1);
    const int* table = block_table + (int64_t)b * max_pages;
    // Behind a window the first keep_first keys stay visible: tiles over [0, sink_end) come first, then the
    // tiles of the window.  Both are aligned to absolute positions, and keys between the two are seen by no
    // query of this block (k_begin is not above any query's window).
    const int sink_end = window > 0 ? min(min(keep_first, k_begin), k_end) : 0;
    const int n_sink = (sink_end + KT - 1) / KT;
    const int n_tiles = n_sink + (k_end > k_begin ? (k_end - k_begin + KT - 1) / KT : 0);

    for (int ti = 0; ti < n_tiles; ++ti) {
        const int kt = ti < n_sink ? ti * KT : k_begin + (ti - n_sink) * KT;
        const int k_lim = ti < n_sink ? sink_end : k_end;
        __syncthreads();                         // the tile before is consumed (first time: Qs, Mx written)
        if (tid < KT) {
            const int kj = kt + tid;
            int s = -1;
            if (kj < k_lim) {
                const int page = table[kj / page_size];
                if (page >= 0) s = page * page_size + kj % page_size;
            }
            slot_of[tid] = s;
        }
        __syncthreads();
        for (int idx = tid; idx < G * KT * dk; idx += 256) {
            const int c = idx % dk, j = (idx / dk) % KT, g = idx / (dk * KT);
            const int s = slot_of[j];
            AT v = from_float<AT>(0.f);
            if (s >= 0) {
                const int page = s / page_size, off = s - page * page_size;
                v = k_cache[(((int64_t)page * G + g) * page_size + off) * dk + c];
            }
            KV[((int64_t)g * KT + j) * ksd + c] = v;
        }
        __syncthreads();
        // raw scores, scaled and capped
        for (int e = tid; e < R * KT; e += 256) {
            const int r = e / KT, j = e - r * KT;
            const int g = (r / QT) / rep;
            const AT* qr = Qs + (int64_t)r * dk;
            const AT* kr = KV + ((int64_t)g * KT + j) * ksd;
            float dot = 0.f;
            for (int c = 0; c < dk; ++c) dot += to_float(qr[c]) * to_float(kr[c]);
            dot *= scale;
            if (cap > 0.f) dot = cap * tanhf(dot / cap);
            S1[r * SP + j] = dot;
        }
        __syncthreads();
        // values of the tile replace its keys while the scores are mixed
        for (int idx = tid; idx < G * KT * dv; idx += 256) {
            const int c = idx % dv, j = (idx / dv) % KT, g = idx / (dv * KT);
            const int s = slot_of[j];
            AT v = from_float<AT>(0.f);
            if (s >= 0) {
                const int page = s / page_size, off = s - page * page_size;
                v = v_cache[(((int64_t)page * G + g) * page_size + off) * vrs + c];
            }
            KV[idx] = v;
        }
        for (int e = tid; e < R * KT; e += 256) {
            const int r = e / KT, j = e - r * KT;
            const int h = r / QT, i = r - h * QT;
            float s;
            if (mix) {
                s = 0.f;
                for (int g = 0; g < H; ++g) s += Mx[h * H + g] * S1[(g * QT + i) * SP + j];
            } else {
                s = S1[r * SP + j];
            }
            const int kj = kt + j, pos = p_lo + i;
            const bool vis = i < nq && kj <= pos && (window == 0 || kj > pos - window || kj < keep_first) &&
                             slot_of[j] >= 0;
            S2[r * SP + j] = vis ? s : -INFINITY;
        }
        __syncthreads();
        // running softmax of this warp's rows, then P.V
#pragma unroll
        for (int m = 0; m < RPW; ++m) {
            const int r = warp * rpw + m;
            if (m < rpw && r < R) {
                float* prow = S2 + r * SP;
                if (head_bias) {
                    // every key weighs in by itself: nothing to rescale, nothing to sum
                    const float hb = head_bias[r / QT];
                    for (int j = lane; j < KT; j += 32)
                        prow[j] = prow[j] == -INFINITY ? 0.f : 1.0f / (1.0f + expf(-(prow[j] + hb)));
                    continue;
                }
                float tmax = -INFINITY;
                for (int j = lane; j < KT; j += 32) tmax = fmaxf(tmax, prow[j]);
                tmax = warp_max(tmax);
                const float m_new = fmaxf(m_run[m], tmax);
                float alpha = 1.f, psum = 0.f;
                if (m_new == -INFINITY) {
                    for (int j = lane; j < KT; j += 32) prow[j] = 0.f;
                } else {
                    alpha = expf(m_run[m] - m_new);
                    for (int j = lane; j < KT; j += 32) {
                        const float p = expf(prow[j] - m_new);
                        prow[j] = p;
                        psum += p;
                    }
                }
                psum = warp_sum(psum);
                l_run[m] = l_run[m] * alpha + psum;
                m_run[m] = m_new;
#pragma unroll
                for (int n = 0; n < CPL; ++n) acc[m][n] *= alpha;
            }
        }
        __syncwarp();
        for (int j = 0; j < KT; ++j) {
            float vv[CPL];
            int g_have = -1;
#pragma unroll
            for (int m = 0; m < RPW; ++m) {
                const int r = warp * rpw + m;
                if (m < rpw && r < R) {
                    if (g_of[m] != g_have) {
                        g_have = g_of[m];
#pragma unroll
                        for (int n = 0; n < CPL; ++n) {
                            const int c = lane + 32 * n;
                            vv[n] = c < dv ? to_float(KV[((int64_t)g_have * KT + j) * dv + c]) : 0.f;
                        }
                    }
                    const float p = S2[r * SP + j];
#pragma unroll
                    for (int n = 0; n < CPL; ++n) acc[m][n] += p * vv[n];
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < RPW; ++m) {
        const int r = warp * rpw + m;
        if (m < rpw && r < R) {
            const int h = r / QT, i = r - h * QT;
            if (i < nq) {
                const float inv = head_bias ? 1.f : (l_run[m] > 0.f ? 1.f / l_run[m] : 0.f);
                AT* o = out + ((int64_t)(q0 + qt * QT + i) * H + h) * dv;
#pragma unroll
                for (int n = 0; n < CPL; ++n) {
                    const int c = lane + 32 * n;
                    if (c < dv) o[c] = from_float<AT>(acc[m][n] * inv);
                }
            }
        }
    }
}

// Queries per block and keys per tile for a model's sizes: as many queries as the rows allow (at most
// 16), and the largest key tile whose buffers fit into shared memory.  A function of the model only.
struct MixPlan { int QT, KT, rpw; size_t smem; bool ok; };

static size_t mix_smem(int H, int G, int dk, int dv, int esize, int qt, int kt) {
    const int R = H * qt;
    const int ksd = dk + (esize == 2 ? 2 : 1);
    const size_t kv = (size_t)G * kt * (ksd > dv ? ksd : dv) * esize;
    return (size_t)2 * R * (kt + 1) * 4 + (size_t)H * H * 4 + (size_t)kt * 4 + (size_t)R * dk * esize + kv + 16;
}

static MixPlan plan_attn_mix(int H, int G, int dk, int dv, int esize, bool decode) {
    MixPlan p = {1, 32, 1, 0, false};
    const int cpl = (dv + 31) / 32;
    const int max_rows = 8 * (cpl >= 8 ? 8 : 16);
    if (H > max_rows) return p;
    int qt = max_rows / H;
    if (qt > 16) qt = 16;
    while (true) {
        for (int kt = 32; kt >= 8; kt /= 2) {
            if (mix_smem(H, G, dk, dv, esize, qt, kt) <= 200 * 1024) {
                // a step of single tokens takes one query per block and the same key tiles
                p.QT = decode ? 1 : qt;
                p.KT = kt;
                p.rpw = (H * p.QT + 7) / 8;
                p.smem = mix_smem(H, G, dk, dv, esize, p.QT, kt);
                p.ok = true;
                return p;
            }
        }
        if (qt == 1) break;
        qt /= 2;
    }
    return p;
}

}  // namespace mi

using namespace mi;

extern "C" {

int mi_rope_store(const float* qkv, const int* positions, const float* inv_freq, const int* slot_mapping,
                  void* q_out, void* k_cache, void* v_cache, int adtype, int T, int nh, int nkv, int dk, int dv,
                  int rot_dim, int page_size, const float* q_gain, const float* k_gain, float eps, int neighbours,
                  const float* v_first, int64_t v_first_stride, const float* lam, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if ((q_gain == nullptr) != (k_gain == nullptr)) {
        set_last_error("rope_store: the gains of the query norm and of the key norm come together");
        return kBadShape;
    }
    if (rot_dim < 0 || rot_dim > dk || rot_dim % 2 || (rot_dim > 0 && !inv_freq)) {
        set_last_error("rope_store: %d rotary dimensions of a head of %d", rot_dim, dk);
        return kBadShape;
    }
    if (v_first && (!lam || v_first_stride < (int64_t)nkv * dv)) {
        set_last_error("rope_store: blended values need their weight and rows of at least %d", nkv * dv);
        return kBadShape;
    }
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                           reinterpret_cast<uintptr_t>(q_gain) | reinterpret_cast<uintptr_t>(k_gain) |
                           reinterpret_cast<uintptr_t>(v_first);
    if (dk % 4 == 0 && dv % 4 == 0 && rot_dim % (neighbours ? 4 : 8) == 0 && dk <= 512 && (ptrs & 15) == 0 &&
        (!v_first || v_first_stride % 4 == 0)) {
        const dim3 grid(T, (nh + 2 * nkv + 7) / 8);
        const size_t smem = sizeof(float) * (rot_dim > 0 ? rot_dim : 1);
#define MI_ROPE_STORE_VEC(CH)                                                                                        \
    MI_DISPATCH_1(adtype, AT,                                                                                        \
        launch_dependent(rope_store_vec_kernel<AT, CH>, grid, dim3(256), smem, stream, qkv, positions, inv_freq,     \
                         slot_mapping, (AT*)q_out, (AT*)k_cache, (AT*)v_cache, nh, nkv, dk, dv, rot_dim, page_size,  \
                         q_gain, k_gain, eps, neighbours, v_first, v_first_stride, lam))
        if (dk <= 128) { MI_ROPE_STORE_VEC(1); }
        else if (dk <= 256) { MI_ROPE_STORE_VEC(2); }
        else { MI_ROPE_STORE_VEC(4); }
#undef MI_ROPE_STORE_VEC
        return finish_launch("rope_store");
    }
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(rope_store_kernel<AT>, dim3(T), dim3(256),
                         sizeof(float) * ((rot_dim > 0 ? rot_dim : 1) + nh + nkv), stream, qkv, positions, inv_freq,
                         slot_mapping, (AT*)q_out, (AT*)k_cache, (AT*)v_cache, nh, nkv, dk, dv, rot_dim, page_size,
                         q_gain, k_gain, eps, neighbours, v_first, v_first_stride, lam));
    return finish_launch("rope_store");
}

// 1 if the sizes are taken
int mi_attn_mix_supported(int H, int G, int dk, int dv, int esize) {
    if (H < 1 || G < 1 || H % G || dk < 1 || dv < 1 || dv > 256) return 0;
    return plan_attn_mix(H, G, dk, dv, esize, false).ok && plan_attn_mix(H, G, dk, dv, esize, true).ok;
}

// head_bias: null, or a number per head that makes every visible key's weight logistic(score + head_bias[h])
// instead of its share of a softmax (then without `sink`)
int mi_attn_mix_form(const void* q, const void* k_cache, const void* v_cache, int adtype, const float* mix,
                     const int* block_table, const int* q_start, const int* kv_len, void* out, int B, int max_q_len,
                     int H, int G, int dk, int dv, int page_size, int max_pages, int window, float scale, float cap,
                     int keep_first, int vrs, int sink, const float* head_bias, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return kOk;
    if (head_bias && sink) {
        set_last_error("mixed-head attention: a key more belongs to a softmax, not to weights that are not normalised");
        return kBadShape;
    }
    if (keep_first < 0 || vrs < dv) {
        set_last_error("mixed-head attention: %d kept first keys, value rows of %d every %d elements", keep_first, dv, vrs);
        return kBadShape;
    }
    if (H < 1 || G < 1 || H % G || dk < 1 || dv < 1 || dv > 256) {
        set_last_error("mixed-head attention: heads %d, key/value heads %d, key size %d, value size %d (at most 256)",
                       H, G, dk, dv);
        return kBadShape;
    }
    const int esize = adtype == kBF16 ? 2 : 4;
    const MixPlan p = plan_attn_mix(H, G, dk, dv, esize, max_q_len == 1);
    if (!p.ok) {
        set_last_error("mixed-head attention: %d heads of key size %d do not fit one block", H, dk);
        return kBadShape;
    }
    if (B > 65535) { set_last_error("mixed-head attention: batch %d exceeds the grid limit", B); return kBadShape; }
    const dim3 grid((max_q_len + p.QT - 1) / p.QT, B);
    const int cpl = (dv + 31) / 32;
#define MI_MIX_LAUNCH(CPL)                                                                                    \
    MI_DISPATCH_1(adtype, AT, {                                                                               \
        cudaFuncSetAttribute(attn_mix_kernel<AT, CPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem); \
        launch_dependent(attn_mix_kernel<AT, CPL>, grid, dim3(256), p.smem, stream, (const AT*)q,            \
                         (const AT*)k_cache, (const AT*)v_cache, mix, block_table, q_start, kv_len, (AT*)out, \
                         H, G, dk, dv, page_size, max_pages, window, scale, cap, p.QT, p.KT, p.rpw,          \
                         keep_first, vrs, sink, head_bias);                                                   \
    })
    if (cpl <= 1) MI_MIX_LAUNCH(1);
    else if (cpl <= 2) MI_MIX_LAUNCH(2);
    else if (cpl <= 4) MI_MIX_LAUNCH(4);
    else MI_MIX_LAUNCH(8);
#undef MI_MIX_LAUNCH
    return finish_launch("attn_mix");
}

int mi_attn_mix(const void* q, const void* k_cache, const void* v_cache, int adtype, const float* mix,
                const int* block_table, const int* q_start, const int* kv_len, void* out, int B, int max_q_len,
                int H, int G, int dk, int dv, int page_size, int max_pages, int window, float scale, float cap,
                int keep_first, int vrs, int sink, cudaStream_t stream) {
    return mi_attn_mix_form(q, k_cache, v_cache, adtype, mix, block_table, q_start, kv_len, out, B, max_q_len, H, G, dk,
                            dv, page_size, max_pages, window, scale, cap, keep_first, vrs, sink, nullptr, stream);
}

}  // extern "C"
