// Head-mixing attention (see attention_mix.cu for the mechanism) on the tensor cores, bfloat16 storage.
//
// A block owns 16 consecutive queries of one request with ALL heads: the scores of a (query, key) pair are
// mixed over the heads before the softmax, so no head can be computed alone.  Per tile of KT keys:
//   1. the tile's values are asked for (cp.async, 16 bytes a piece, a buffer of their own); its keys, asked for
//      while the tile before was finished, have landed
//   2. S_h = Q_h K_g^T with mma.sync m16n8k16 (warp w owns heads w, w + 8, ...), scaled, capped, to shared
//      memory as float
//   3. the next tile's keys are asked for; meanwhile the mix over heads and the mask, pair by pair, into a
//      second buffer
//   4. running softmax in the layout of the A fragments (a row's maximum and sum live in a quad of lanes),
//      O_h += P_h V_g with V fragments fetched by ldmatrix.trans from the row-major tile
// Behind a window the first keep_first keys of a request stay visible; a value row may be the leading part of
// a longer row (`vrs` elements from one token's values to the next one's).
// Steps of one token per request are split over the keys (blocks of 64 keys write a partial maximum, sum
// and unnormalised output; a merge kernel finishes), since one block per request cannot pull a window of
// keys from memory fast enough.
//
// With `head_bias` (a number per head) there is no softmax: a visible key's weight is logistic(score + head_bias[h]),
// not normalised over the keys, so nothing is rescaled and the partial results of a split step are simply added.
//
// Built for value sizes 64 and 128 and key sizes that are multiples of 16.  The accumulators of 16 heads of
// value size 128 (32 of 64) fill one block's registers; with more heads several blocks share a query tile,
// each forming all heads' scores and finishing its own group of heads.  Shapes whose tiles do not fit shared
// memory, other sizes and the float path take the kernel of attention_mix.cu.

#include "common.cuh"

namespace mi {

__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// tanh and exp of the bfloat16 path: the hardware's exponential (a few units in the last place), where the
// library functions cost thirty to forty instructions apiece, a third of a key tile's work
__device__ __forceinline__ float fast_tanh(float x) { return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f); }

__device__ __forceinline__ void tile_copy_16(void* smem_dst, const void* src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void tile_copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void tile_copy_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

constexpr int kTcQ = 16;          // queries per block
constexpr int kTcWarps = 8;
constexpr int kTcSplitKeys = 64;  // keys per block of a split step

template <int HPW, int NT, int KT>      // heads per warp, value size / 8, keys per tile
__global__ void __launch_bounds__(256, 1)
attn_mix_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, const float* __restrict__ mix,
                   const int* __restrict__ block_table, const int* __restrict__ q_start,
                   const int* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int H, int G, int dk, int page_size, int max_pages, int window,
                   float scale, float cap, int splits, int hgroups, int keep_first, int vrs, int sink,
                   const float* __restrict__ head_bias) {
    constexpr int DV = NT * 8;
    constexpr int SP = KT + 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    wait_for_earlier_kernels();
    // with more heads than one block's registers hold accumulators for, `hgroups` blocks share a query tile:
    // each forms all heads' scores (the mix needs them) and finishes the heads [h_lo, h_hi) only
    const int b = blockIdx.y, qt = blockIdx.x / hgroups, hg = blockIdx.x % hgroups, split = blockIdx.z;
    const int HG = (H + hgroups - 1) / hgroups;
    const int h_lo = hg * HG, h_hi = min(H, h_lo + HG);
    const int q0 = q_start[b], q_len = q_start[b + 1] - q0;
    if (qt * kTcQ >= q_len) return;
    const int kvl = kv_len[b];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = lane >> 2, c2 = (lane & 3) * 2;
    const int rep = H / G;
    const int dkp = dk + 8, dvp = DV + 8;
    float* S1 = reinterpret_cast<float*>(smem_raw);                       // [H][16][SP]
    float* S2 = S1 + H * kTcQ * SP;                                       // [HG][16][SP], heads of this block
    float* Mx = S2 + HG * kTcQ * SP;                                      // [H][H]
    int* slots = reinterpret_cast<int*>(Mx + ((H * H + 3) & ~3));         // [2][KT]: this tile's and the next one's
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(slots + 2 * KT); // [H][16][dkp]
    __nv_bfloat16* Kb = Qs + (size_t)H * kTcQ * dkp;                      // [G][KT][dkp]
    __nv_bfloat16* Vb = Kb + (size_t)G * KT * dkp;                        // [G][KT][dvp]

    const int nq = min(kTcQ, q_len - qt * kTcQ);
    const int p_lo = kvl - q_len + qt * kTcQ;
    const int p_hi = p_lo + nq - 1;

    // Q tile: rows of 16 bytes
    const int qchunks = dk / 8;
    for (int idx = tid; idx < H * kTcQ * qchunks; idx += 256) {
        const int c8 = idx % qchunks, i = (idx / qchunks) % kTcQ, h = idx / (qchunks * kTcQ);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < nq) v = *reinterpret_cast<const uint4*>(q + ((size_t)(q0 + qt * kTcQ + i) * H + h) * dk + c8 * 8);
        *reinterpret_cast<uint4*>(Qs + ((size_t)h * kTcQ + i) * dkp + c8 * 8) = v;
    }
    // transposed: Mx[g * H + h] = mix[h][g], so that four heads' weights of one g are one 16-byte read
    if (mix) for (int idx = tid; idx < H * H; idx += 256) Mx[(idx % H) * H + idx / H] = mix[idx];

    float acc[HPW][NT][4];
    float m_run[HPW][2], l_run[HPW][2];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        // a key more of score 0 and no value (`sink`): of an unsplit step the running maximum starts at 0 and
        // the running sum at 1 (in one lane of the quad that shares a row); a split step leaves it to the merge
        const bool sunk = sink && splits == 1;
        m_run[hh][0] = m_run[hh][1] = sunk ? 0.f : -INFINITY;
        l_run[hh][0] = l_run[hh][1] = (sunk && (lane & 3) == 0) ? 1.f : 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[hh][nt][x] = 0.f;
    }

    int k_begin = 0;
    if (window > 0) k_begin = max(0, p_lo - window + 1);
    k_begin = (k_begin / KT) * KT;
    int k_end = min(kvl, p_hi + 1);
    // behind a window the first keep_first keys stay visible: tiles over [0, sink_end) come before the
    // window's tiles (see attention_mix.cu); of a split step the last block takes them
    int sink_end = window > 0 ? min(min(keep_first, k_begin), k_end) : 0;
    if (splits > 1) {
        if (keep_first > 0 && split == splits - 1) {
            k_begin = k_end;                     // the kept first keys alone
        } else {
            sink_end = 0;
            k_begin += split * kTcSplitKeys;
            k_end = min(k_end, k_begin + kTcSplitKeys);
        }
    }
    const int n_sink = (sink_end + KT - 1) / KT;
    const int n_tiles = n_sink + (k_end > k_begin ? (k_end - k_begin + KT - 1) / KT : 0);
    auto tile_start = [&](int ti) { return ti < n_sink ? ti * KT : k_begin + (ti - n_sink) * KT; };
    auto tile_limit = [&](int ti) { return ti < n_sink ? sink_end : k_end; };
    const int* table = block_table + (size_t)b * max_pages;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    // Keys and values travel a step ahead of their use (cp.async): the values of a tile are asked for before its
    // scores are formed, the keys of the next tile as soon as the scores have left the key buffer.
    constexpr int vchunks = DV / 8;
    auto find_slots = [&](int ti, int* slot_of) {
        if (tid < KT) {
            const int kj = tile_start(ti) + tid;
            int s = -1;
            if (kj < tile_limit(ti)) {
                const int page = table[kj / page_size];
                if (page >= 0) s = page * page_size + kj % page_size;
            }
            slot_of[tid] = s;
        }
    };
    auto fetch_keys = [&](const int* slot_of) {
        for (int idx = tid; idx < G * KT * qchunks; idx += 256) {
            const int c8 = idx % qchunks, j = (idx / qchunks) % KT, g = idx / (qchunks * KT);
            const int s = slot_of[j];
            __nv_bfloat16* dst = Kb + ((size_t)g * KT + j) * dkp + c8 * 8;
            if (s >= 0) {
                const int page = s / page_size, off = s - page * page_size;
                tile_copy_16(dst, k_cache + (((size_t)page * G + g) * page_size + off) * dk + c8 * 8);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto fetch_values = [&](const int* slot_of) {
        for (int idx = tid; idx < G * KT * vchunks; idx += 256) {
            const int c8 = idx % vchunks, j = (idx / vchunks) % KT, g = idx / (vchunks * KT);
            const int s = slot_of[j];
            __nv_bfloat16* dst = Vb + ((size_t)g * KT + j) * dvp + c8 * 8;
            if (s >= 0) {
                const int page = s / page_size, off = s - page * page_size;
                tile_copy_16(dst, v_cache + (((size_t)page * G + g) * page_size + off) * vrs + c8 * 8);
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (n_tiles > 0) {
        find_slots(0, slots);
        __syncthreads();
        fetch_keys(slots);
    }
    tile_copy_commit();
    int which = 0;
    for (int ti = 0; ti < n_tiles; ++ti, which ^= 1) {
        const int kt = tile_start(ti);
        const int* slot_of = slots + which * KT;
        __syncthreads();                         // the tile before has left the value buffer and its scores
        fetch_values(slot_of);
        tile_copy_commit();
        if (ti + 1 < n_tiles) find_slots(ti + 1, slots + (which ^ 1) * KT);
        tile_copy_wait_but_one();                // this tile's keys
        __syncthreads();
        // ---- scores of all heads ----
        for (int h = warp; h < H; h += kTcWarps) {
            {
                const int g = h / rep;
                float c[KT / 8][4];
#pragma unroll
                for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
                    for (int x = 0; x < 4; ++x) c[nt][x] = 0.f;
                const __nv_bfloat16* qb = Qs + (size_t)h * kTcQ * dkp;
                const __nv_bfloat16* kb = Kb + (size_t)g * KT * dkp;
                for (int ks = 0; ks < dk; ks += 16) {
                    const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qb + r0 * dkp + ks + c2);
                    const uint32_t a1 = *reinterpret_cast<const uint32_t*>(qb + (r0 + 8) * dkp + ks + c2);
                    const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qb + r0 * dkp + ks + 8 + c2);
                    const uint32_t a3 = *reinterpret_cast<const uint32_t*>(qb + (r0 + 8) * dkp + ks + 8 + c2);
#pragma unroll
                    for (int nt = 0; nt < KT / 8; ++nt) {
                        const __nv_bfloat16* kr = kb + (size_t)(nt * 8 + r0) * dkp + ks + c2;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
                        mma_bf16_16816(c[nt], a0, a1, a2, a3, b0, b1);
                    }
                }
                float* sb = S1 + (size_t)h * kTcQ * SP;
#pragma unroll
                for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        float s = c[nt][x] * scale;
                        if (cap > 0.f) s = cap * fast_tanh(s * inv_cap);
                        sb[(r0 + (x >> 1) * 8) * SP + nt * 8 + c2 + (x & 1)] = s;
                    }
            }
        }
        __syncthreads();
        // ---- the next tile's keys set off; mix and mask ----
        if (ti + 1 < n_tiles) fetch_keys(slots + (which ^ 1) * KT);
        tile_copy_commit();
        for (int e = tid; e < kTcQ * KT; e += 256) {
            const int i = e / KT, j = e - i * KT;
            const int kj = kt + j, pos = p_lo + i;
            const bool vis = i < nq && kj <= pos && (window == 0 || kj > pos - window || kj < keep_first) &&
                             slot_of[j] >= 0;
            if (!vis) {
                for (int h = h_lo; h < h_hi; ++h) S2[((h - h_lo) * kTcQ + i) * SP + j] = -INFINITY;
            } else if (!mix) {
                for (int h = h_lo; h < h_hi; ++h) S2[((h - h_lo) * kTcQ + i) * SP + j] = S1[(h * kTcQ + i) * SP + j];
            } else if (((H | HG) & 3) == 0) {
                for (int h = h_lo; h < h_hi; h += 4) {
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
                    for (int g = 0; g < H; ++g) {
                        const float v = S1[(g * kTcQ + i) * SP + j];
                        const float4 w = *reinterpret_cast<const float4*>(Mx + g * H + h);
                        s0 += w.x * v; s1 += w.y * v; s2 += w.z * v; s3 += w.w * v;
                    }
                    S2[((h - h_lo) * kTcQ + i) * SP + j] = s0;
                    S2[((h - h_lo + 1) * kTcQ + i) * SP + j] = s1;
                    S2[((h - h_lo + 2) * kTcQ + i) * SP + j] = s2;
                    S2[((h - h_lo + 3) * kTcQ + i) * SP + j] = s3;
                }
            } else {
                for (int h = h_lo; h < h_hi; ++h) {
                    float s = 0.f;
                    for (int g = 0; g < H; ++g) s += Mx[g * H + h] * S1[(g * kTcQ + i) * SP + j];
                    S2[((h - h_lo) * kTcQ + i) * SP + j] = s;
                }
            }
        }
        tile_copy_wait_but_one();                // this tile's values
        __syncthreads();
        // ---- softmax and P.V of this block's heads ----
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int h = h_lo + warp + kTcWarps * hh;
            if (h < h_hi) {
                const int g = h / rep;
                const float* sb = S2 + (size_t)(h - h_lo) * kTcQ * SP;
                float p[KT / 8][4];
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < KT / 8; ++nt) {
                    p[nt][0] = sb[r0 * SP + nt * 8 + c2];
                    p[nt][1] = sb[r0 * SP + nt * 8 + c2 + 1];
                    p[nt][2] = sb[(r0 + 8) * SP + nt * 8 + c2];
                    p[nt][3] = sb[(r0 + 8) * SP + nt * 8 + c2 + 1];
                    mx0 = fmaxf(mx0, fmaxf(p[nt][0], p[nt][1]));
                    mx1 = fmaxf(mx1, fmaxf(p[nt][2], p[nt][3]));
                }
                if (head_bias) {
                    // every key weighs in by itself (a masked score of -inf gives 0): nothing to rescale
                    const float hb = head_bias[h];
#pragma unroll
                    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            p[nt][x] = p[nt][x] == -INFINITY ? 0.f : __fdividef(1.0f, 1.0f + __expf(-(p[nt][x] + hb)));
                } else {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m_run[hh][0], mx0), mn1 = fmaxf(m_run[hh][1], mx1);
                const float al0 = mn0 == -INFINITY ? 1.f : __expf(m_run[hh][0] - mn0);
                const float al1 = mn1 == -INFINITY ? 1.f : __expf(m_run[hh][1] - mn1);
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int nt = 0; nt < KT / 8; ++nt) {
                    p[nt][0] = mn0 == -INFINITY ? 0.f : __expf(p[nt][0] - mn0);
                    p[nt][1] = mn0 == -INFINITY ? 0.f : __expf(p[nt][1] - mn0);
                    p[nt][2] = mn1 == -INFINITY ? 0.f : __expf(p[nt][2] - mn1);
                    p[nt][3] = mn1 == -INFINITY ? 0.f : __expf(p[nt][3] - mn1);
                    s0 += p[nt][0] + p[nt][1];
                    s1 += p[nt][2] + p[nt][3];
                }
                l_run[hh][0] = l_run[hh][0] * al0 + s0;     // a lane's share; the quad is summed at the end
                l_run[hh][1] = l_run[hh][1] * al1 + s1;
                m_run[hh][0] = mn0;
                m_run[hh][1] = mn1;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    acc[hh][nt][0] *= al0; acc[hh][nt][1] *= al0;
                    acc[hh][nt][2] *= al1; acc[hh][nt][3] *= al1;
                }
                }
                const __nv_bfloat16* vb = Vb + (size_t)g * KT * dvp;
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk) {
                    const uint32_t a0 = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
                    const uint32_t a1 = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
                    const uint32_t a2 = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
                    const uint32_t a3 = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
                    const __nv_bfloat16* vrow = vb + (size_t)(kk * 16 + (lane & 15)) * dvp;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        uint32_t b0, b1;
                        ldmatrix_x2_trans(b0, b1, vrow + nt * 8);
                        mma_bf16_16816(acc[hh][nt], a0, a1, a2, a3, b0, b1);
                    }
                }
            }
        }
    }
    // ---- results ----
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int h = h_lo + warp + kTcWarps * hh;
        if (h < h_hi) {
            float l0 = l_run[hh][0], l1 = l_run[hh][1];
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            if (splits > 1) {
                // one query per request: row 0 of the tile
                if (r0 == 0) {
                    const size_t base = ((size_t)b * splits + split) * H + h;
                    float* po = part_o + base * DV;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        po[nt * 8 + c2] = acc[hh][nt][0];
                        po[nt * 8 + c2 + 1] = acc[hh][nt][1];
                    }
                    if ((lane & 3) == 0) { part_ml[base * 2] = m_run[hh][0]; part_ml[base * 2 + 1] = l0; }
                }
            } else {
                const float i0 = head_bias ? 1.f : (l0 > 0.f ? 1.f / l0 : 0.f);
                const float i1 = head_bias ? 1.f : (l1 > 0.f ? 1.f / l1 : 0.f);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (r0 < nq)
                        *reinterpret_cast<uint32_t*>(out + ((size_t)(q0 + qt * kTcQ + r0) * H + h) * DV + nt * 8 + c2) =
                            pack_bf16(acc[hh][nt][0] * i0, acc[hh][nt][1] * i0);
                    if (r0 + 8 < nq)
                        *reinterpret_cast<uint32_t*>(out + ((size_t)(q0 + qt * kTcQ + r0 + 8) * H + h) * DV + nt * 8 + c2) =
                            pack_bf16(acc[hh][nt][2] * i1, acc[hh][nt][3] * i1);
                }
            }
        }
    }
}

// out[b, h, :] from the partial results of the splits, in split order.  The splits' maxima and sums are fetched
// once, all at a time, and every split's weight exp(m_s - m) is formed once for all columns.
constexpr int kMergeMaxSplits = 12288;          // two floats a split in shared memory: 96 KiB
__global__ void __launch_bounds__(128)
attn_mix_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                      const int* __restrict__ q_start, __nv_bfloat16* __restrict__ out, int H, int DV, int splits,
                      int sink, int plain_sum) {
    extern __shared__ float merge_sh[];         // [splits] weights, [splits] sums
    float* wgt = merge_sh;
    float* lsum = merge_sh + splits;
    wait_for_earlier_kernels();
    const int b = blockIdx.y, h = blockIdx.x;
    if (plain_sum) {
        // weights that are not normalised: the splits' partial outputs are added as they are, in split order
        const int row0 = q_start[b];
        for (int c = threadIdx.x; c < DV; c += blockDim.x) {
            float o = 0.f;
            for (int s = 0; s < splits; ++s) o += part_o[(((size_t)b * splits + s) * H + h) * DV + c];
            out[((size_t)row0 * H + h) * DV + c] = __float2bfloat16_rn(o);
        }
        return;
    }
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (((size_t)b * splits + s) * H + h) * 2);
        wgt[s] = ml.x;
        lsum[s] = ml.y;
    }
    __syncthreads();
    float m = sink ? 0.f : -INFINITY;           // the key of score 0 that `sink` adds counts here, once
    for (int s = 0; s < splits; ++s) m = fmaxf(m, wgt[s]);
    __syncthreads();
    for (int s = threadIdx.x; s < splits; s += blockDim.x) wgt[s] = wgt[s] == -INFINITY ? 0.f : expf(wgt[s] - m);
    __syncthreads();
    float l = sink ? expf(-m) : 0.f;
    for (int s = 0; s < splits; ++s) l += lsum[s] * wgt[s];        // in split order
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int row = q_start[b];
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float w = wgt[s];
            if (w != 0.f) o += part_o[(((size_t)b * splits + s) * H + h) * DV + c] * w;
        }
        out[((size_t)row * H + h) * DV + c] = __float2bfloat16_rn(o * inv);
    }
}

static size_t tc_smem(int H, int HG, int G, int dk, int dv, int kt) {
    const int dkp = dk + 8, dvp = dv + 8;
    return (size_t)(H + HG) * kTcQ * (kt + 1) * 4 + (size_t)((H * H + 3) & ~3) * 4 + (size_t)2 * kt * 4 +
           (size_t)H * kTcQ * dkp * 2 + (size_t)G * kt * (dkp + dvp) * 2 + 16;
}

struct TcPlan { int kt, hgroups, hpw; };

// keys per tile, blocks per query tile and heads per warp for a model's sizes (kt 0: the shape is not taken)
static TcPlan tc_plan(int H, int G, int dk, int dv) {
    TcPlan p = {0, 1, 1};
    if (H < 1 || G < 1 || H % G || dk % 16 || dk < 16 || dk > 256 || (dv != 64 && dv != 128)) return p;
    const int max_hpw = 32 / (dv / 8);                  // accumulators of a warp: hpw * dv / 8 * 4 registers a lane
    int hgroups = 1;
    while (((H + hgroups - 1) / hgroups + kTcWarps - 1) / kTcWarps > max_hpw) ++hgroups;
    const int HG = (H + hgroups - 1) / hgroups;
    p.hgroups = hgroups;
    p.hpw = (HG + kTcWarps - 1) / kTcWarps;
    if (tc_smem(H, HG, G, dk, dv, 32) <= 220 * 1024) p.kt = 32;
    else if (tc_smem(H, HG, G, dk, dv, 16) <= 220 * 1024) p.kt = 16;
    return p;
}

}  // namespace mi

using namespace mi;

extern "C" {

int mi_attn_mix_tc_supported(int H, int G, int dk, int dv) { return tc_plan(H, G, dk, dv).kt > 0; }

// splits a step of single tokens is cut into, given the longest span of keys a query can see
int mi_attn_mix_tc_splits(int span) { return (span + kTcSplitKeys - 1) / kTcSplitKeys + 1; }

int mi_attn_mix_tc_form(const void* q, const void* k_cache, const void* v_cache, const float* mix,
                        const int* block_table, const int* q_start, const int* kv_len, void* out, float* part_o,
                        float* part_ml, int B, int max_q_len, int H, int G, int dk, int dv, int page_size,
                        int max_pages, int window, float scale, float cap, int splits, int keep_first, int vrs,
                        int sink, const float* head_bias, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return kOk;
    if (head_bias && sink) {
        set_last_error("mixed-head attention (tensor cores): a key more belongs to a softmax, not to weights that are not normalised");
        return kBadShape;
    }
    if (keep_first < 0 || vrs < dv || vrs % 8) {
        set_last_error("mixed-head attention (tensor cores): %d kept first keys, value rows of %d every %d elements",
                       keep_first, dv, vrs);
        return kBadShape;
    }
    const TcPlan plan = tc_plan(H, G, dk, dv);
    const int kt = plan.kt;
    if (!kt) {
        set_last_error("mixed-head attention (tensor cores): heads %d/%d, key size %d, value size %d are not taken", H, G, dk, dv);
        return kBadShape;
    }
    if (splits < 1 || (splits > 1 && (max_q_len != 1 || !part_o || !part_ml)) || B > 65535 || splits > kMergeMaxSplits) {
        set_last_error("mixed-head attention (tensor cores): %d splits with portions of %d tokens, batch %d", splits, max_q_len, B);
        return kBadShape;
    }
    const int hpw = plan.hpw, hgroups = plan.hgroups;
    const size_t smem = tc_smem(H, (H + hgroups - 1) / hgroups, G, dk, dv, kt);
    const dim3 grid(((max_q_len + kTcQ - 1) / kTcQ) * hgroups, B, splits);
#define MI_TC_LAUNCH(HPW, NT, KT)                                                                               \
    do {                                                                                                        \
        cudaFuncSetAttribute(attn_mix_tc_kernel<HPW, NT, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_dependent(attn_mix_tc_kernel<HPW, NT, KT>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)q, \
                         (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, mix, block_table, q_start, \
                         kv_len, (__nv_bfloat16*)out, part_o, part_ml, H, G, dk, page_size, max_pages, window,  \
                         scale, cap, splits, hgroups, keep_first, vrs, sink, head_bias);                        \
    } while (0)
#define MI_TC_KT(HPW, NT) do { if (kt == 32) MI_TC_LAUNCH(HPW, NT, 32); else MI_TC_LAUNCH(HPW, NT, 16); } while (0)
    if (dv == 128) {
        if (hpw == 1) MI_TC_KT(1, 16); else MI_TC_KT(2, 16);
    } else {
        if (hpw == 1) MI_TC_KT(1, 8); else if (hpw == 2) MI_TC_KT(2, 8); else MI_TC_KT(4, 8);
    }
#undef MI_TC_KT
#undef MI_TC_LAUNCH
    int launched = 1;
    if (splits > 1) {
        const size_t merge_smem = (size_t)2 * splits * sizeof(float);
        if (merge_smem > 48 * 1024)
            cudaFuncSetAttribute(attn_mix_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)merge_smem);
        launch_dependent(attn_mix_merge_kernel, dim3(H, B), dim3(128), merge_smem, stream, (const float*)part_o,
                         (const float*)part_ml, q_start, (__nv_bfloat16*)out, H, dv, splits, sink,
                         head_bias ? 1 : 0);
        launched = 2;
    }
    return finish_launch("attn_mix_tc", launched);
}

int mi_attn_mix_tc(const void* q, const void* k_cache, const void* v_cache, const float* mix, const int* block_table,
                   const int* q_start, const int* kv_len, void* out, float* part_o, float* part_ml, int B,
                   int max_q_len, int H, int G, int dk, int dv, int page_size, int max_pages, int window,
                   float scale, float cap, int splits, int keep_first, int vrs, int sink, cudaStream_t stream) {
    return mi_attn_mix_tc_form(q, k_cache, v_cache, mix, block_table, q_start, kv_len, out, part_o, part_ml, B,
                               max_q_len, H, G, dk, dv, page_size, max_pages, window, scale, cap, splits, keep_first,
                               vrs, sink, nullptr, stream);
}

}  // extern "C"
