// Row-wise kernels of residual arrangements other than "norm, part, add, norm, part, add":
//
//   add2_rmsnorm_scalar   hidden += a + b (both optional), then ONE root mean square per row and two
//                         outputs that differ by a scalar gain only: the two norms of a block whose mixer
//                         and feed-forward read the same residual, when each norm's weight is one number
//   geglu_tanh            out = gelu_tanh(gate) * up, gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   clamped_glu           out = g s(a g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit),
//                         s the logistic function: a gated unit whose two halves are bounded before they meet
//   concat_cast           out[t] = [hidden[t] + a[t] + b[t] | other[t]] in the activation type: the input
//                         of a projection that reads the residual beside a second stream
//   rows_plus_vec         hidden[t] = y[t] + vec: a projection's result becomes the residual, plus one row
//   group_rmsnorm         out[t] = hidden[t] / rms * w with the root mean square taken over each of `groups` equal
//                         consecutive parts of the row by itself (out_norm_add takes `groups` as well)
//   out_norm_add          hidden[t] += mult * y[t] / rms(y[t]) * w, and the new row once more in the activation
//                         type: a block whose parts read the residual itself and whose OUTPUT is normalised;
//                         y may be a sum of rows that is formed here and never written out
//   softcap_rows          z <- cap * tanh(z / cap) in place (capped logits)

#include "common.cuh"

namespace mi {

template <typename AT>
__global__ void __launch_bounds__(256)
add2_rmsnorm_scalar_kernel(float* __restrict__ hidden, const float* __restrict__ a, const float* __restrict__ b,
                           const int* __restrict__ rows, const float* __restrict__ gain1,
                           const float* __restrict__ gain2, AT* __restrict__ out1, AT* __restrict__ out2, int H,
                           float eps) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* h = hidden + (int64_t)src * H;
    const float* pa = a ? a + (int64_t)src * H : nullptr;
    const float* pb = b ? b + (int64_t)src * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = h[i];
        if (pa || pb) {
            float dlt = pa ? pa[i] : 0.f;
            if (pb) dlt += pb[i];
            v += dlt;
            if (!rows) h[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)H + eps);
    const float g1 = gain1[0], g2 = gain2 ? gain2[0] : 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = h[i];
        if (rows && (pa || pb)) {
            float dlt = pa ? pa[i] : 0.f;
            if (pb) dlt += pb[i];
            v += dlt;
        }
        const float nv = v * rr;
        out1[(int64_t)r * H + i] = from_float<AT>(nv * g1);
        if (out2) out2[(int64_t)r * H + i] = from_float<AT>(nv * g2);
    }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename AT>
__global__ void geglu_tanh_kernel(const AT* __restrict__ gu, AT* __restrict__ out, int64_t total, int I) {
    wait_for_earlier_kernels();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_float(gu[t * 2 * I + i]);
        const float u = to_float(gu[t * 2 * I + I + i]);
        out[idx] = from_float<AT>(gelu_tanh_f(g) * u);
    }
}

// gate and up halves of float rows [T, 2 I] -> [T, I] in the activation type
template <typename AT>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, AT* __restrict__ out, int64_t total, int I,
                                   float limit, float slope) {
    wait_for_earlier_kernels();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / I;
        const int i = (int)(idx - t * I);
        out[idx] = from_float<AT>(clamped_glu_f(gu[t * 2 * I + i], gu[t * 2 * I + I + i], limit, slope));
    }
}

// bfloat16 rows with I a multiple of 8: 16 bytes per load and store
__global__ void geglu_tanh_bf16x8_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, int64_t total_vec,
                                         int Iv) {
    wait_for_earlier_kernels();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / Iv;
        const int i = (int)(idx - t * Iv);
        const uint4 gv = __ldg(gu + t * 2 * Iv + i);
        const uint4 uv = __ldg(gu + t * 2 * Iv + Iv + i);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 r;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            r2[j] = __floats2bfloat162_rn(gelu_tanh_f(g.x) * u.x, gelu_tanh_f(g.y) * u.y);
        }
        out[idx] = r;
    }
}

template <typename AT>
__global__ void __launch_bounds__(256)
concat_cast_kernel(const float* __restrict__ hidden, const float* __restrict__ a, const float* __restrict__ b,
                   const float* __restrict__ other, AT* __restrict__ out, int H) {
    wait_for_earlier_kernels();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hidden[t * H + i];
        if (a || b) {
            float dlt = a ? a[t * H + i] : 0.f;
            if (b) dlt += b[t * H + i];
            v += dlt;
        }
        out[t * 2 * H + i] = from_float<AT>(v);
        out[t * 2 * H + H + i] = from_float<AT>(other[t * H + i]);
    }
}

template <typename WT>
__global__ void __launch_bounds__(256)
rows_plus_vec_kernel(float* __restrict__ hidden, const float* __restrict__ y, const WT* __restrict__ vec, int H) {
    wait_for_earlier_kernels();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) hidden[t * H + i] = y[t * H + i] + to_float(vec[i]);
}

// y[t] = sum_k wk[t, k] * rows[index[t, k]] + scale[t] * extra[t], or a tensor as it is.  `wk` null: weights of
// one; `index` null: rows t * K + k.  Added in slot order, the extra term last.
struct RowSum {
    const float* y;         // [T, H] or null
    const float* rows;      // [N, H]
    const int* index;       // [T, K] or null
    const float* wk;        // [T, K] or null
    const float* extra;     // [T, H] or null
    const float* scale;     // [T] (with extra)
    int K;
};

__device__ __forceinline__ float row_sum_at(const RowSum& s, int64_t t, int i, int H) {
    if (s.y) return s.y[t * H + i];
    float v = 0.f;
    for (int k = 0; k < s.K; ++k) {
        const int64_t r = s.index ? s.index[t * s.K + k] : t * s.K + k;
        const float x = s.rows[r * H + i];
        v += s.wk ? s.wk[t * s.K + k] * x : x;
    }
    if (s.extra) v += s.scale[t] * s.extra[t * H + i];
    return v;
}

// One block per row and group of columns (gs = H / groups columns from blockIdx.y * gs on; one group: the whole
// row).  The sum of squares runs in an order that depends on gs only.
template <typename AT, typename WT>
__global__ void __launch_bounds__(256)
out_norm_add_kernel(float* __restrict__ hidden, RowSum s, const WT* __restrict__ w, AT* __restrict__ x_out, int H,
                    float eps, float mult, int gs) {
    extern __shared__ float yrow[];             // [gs] when it fits (else the sum is formed twice)
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int64_t t = blockIdx.x;
    const int c0 = blockIdx.y * gs;
    const bool staged = gs <= 8192;
    float ss = 0.f;
    for (int i = c0 + threadIdx.x; i < c0 + gs; i += blockDim.x) {
        const float v = row_sum_at(s, t, i, H);
        if (staged) yrow[i - c0] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)gs + eps);
    for (int i = c0 + threadIdx.x; i < c0 + gs; i += blockDim.x) {
        const float v = staged ? yrow[i - c0] : row_sum_at(s, t, i, H);
        const float h = hidden[t * H + i] + mult * (v * rr * to_float(w[i]));
        hidden[t * H + i] = h;
        if (x_out) x_out[t * H + i] = from_float<AT>(h);
    }
}

// Rows of H = 4 n floats on 16-byte boundaries: a thread keeps VPT groups of four of the summed row in
// registers between the sum of squares and the update (H <= 1024 VPT), 16 bytes a load.
__device__ __forceinline__ void axpy4(float4& a, float w, const float4& x) {
    a.x += w * x.x; a.y += w * x.y; a.z += w * x.z; a.w += w * x.w;
}

template <typename AT, typename WT, int VPT>
__global__ void __launch_bounds__(256)
out_norm_add_vec_kernel(float* __restrict__ hidden, RowSum s, const WT* __restrict__ w, AT* __restrict__ x_out, int H,
                        float eps, float mult, int gs) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int64_t t = blockIdx.x;
    const int c0 = blockIdx.y * gs;             // this block's group of gs columns (one group: the whole row)
    const int nv = gs >> 2;
    float4 y[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) y[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (s.y) {
        const float4* yv = reinterpret_cast<const float4*>(s.y + t * H + c0);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + blockDim.x * j;
            if (i < nv) y[j] = yv[i];
        }
    } else {
        for (int k = 0; k < s.K; ++k) {
            const int64_t r = s.index ? s.index[t * s.K + k] : t * s.K + k;
            const float wk = s.wk ? s.wk[t * s.K + k] : 1.0f;
            const float4* rv = reinterpret_cast<const float4*>(s.rows + r * H + c0);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i = threadIdx.x + blockDim.x * j;
                if (i < nv) axpy4(y[j], wk, rv[i]);
            }
        }
        if (s.extra) {
            const float g = s.scale[t];
            const float4* ev = reinterpret_cast<const float4*>(s.extra + t * H + c0);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i = threadIdx.x + blockDim.x * j;
                if (i < nv) axpy4(y[j], g, ev[i]);
            }
        }
    }
    // the residual row is on its way while the squares are added
    float4* hv = reinterpret_cast<float4*>(hidden + t * H + c0);
    float4 h[VPT];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + blockDim.x * j;
        h[j] = i < nv ? hv[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += y[j].x * y[j].x;
        ss += y[j].y * y[j].y;
        ss += y[j].z * y[j].z;
        ss += y[j].w * y[j].w;
    }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + blockDim.x * j;
        if (i < nv) {
            const int c = c0 + 4 * i;
            h[j].x += mult * (y[j].x * rr * to_float(w[c]));
            h[j].y += mult * (y[j].y * rr * to_float(w[c + 1]));
            h[j].z += mult * (y[j].z * rr * to_float(w[c + 2]));
            h[j].w += mult * (y[j].w * rr * to_float(w[c + 3]));
            hv[i] = h[j];
            if (x_out) store4(x_out + t * H + c, h[j]);
        }
    }
}

// out[n, :] = x[row, :] / rms * w with the root mean square of each group of gs columns by itself; one block per
// (row, group).  `rows` (or null) picks the rows of x that are wanted.  The squares are added per thread in
// ascending order and then over the block: an order that depends on gs only.
template <typename OT, typename WT>
__global__ void __launch_bounds__(256)
group_rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const WT* __restrict__ w,
                     OT* __restrict__ out, int H, int gs, float eps, bool vec) {
    __shared__ float scratch[32];
    wait_for_earlier_kernels();
    const int64_t n = blockIdx.x, t = rows ? rows[n] : n;
    const int c0 = blockIdx.y * gs;
    const float* xr = x + t * H + c0;
    OT* orow = out + n * H + c0;
    float ss = 0.f;
    if (vec) {
        for (int i = 4 * threadIdx.x; i < gs; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
    } else {
        for (int i = threadIdx.x; i < gs; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
    }
    ss = block_sum(ss, scratch);
    const float rr = 1.0f / sqrtf(ss / (float)gs + eps);
    if (vec) {
        for (int i = 4 * threadIdx.x; i < gs; i += 4 * blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(xr + i);
            v.x = v.x * rr * to_float(w[c0 + i]);
            v.y = v.y * rr * to_float(w[c0 + i + 1]);
            v.z = v.z * rr * to_float(w[c0 + i + 2]);
            v.w = v.w * rr * to_float(w[c0 + i + 3]);
            store4(orow + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < gs; i += blockDim.x) orow[i] = from_float<OT>(xr[i] * rr * to_float(w[c0 + i]));
    }
}

__global__ void softcap_rows_kernel(float* __restrict__ z, int64_t total, float cap) {
    wait_for_earlier_kernels();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x)
        z[idx] = cap * tanhf(z[idx] / cap);
}

template <typename AT>
__global__ void cast_rows_kernel(const float* __restrict__ x, AT* __restrict__ out, int64_t total) {
    wait_for_earlier_kernels();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x)
        out[idx] = from_float<AT>(x[idx]);
}

}  // namespace mi

using namespace mi;

extern "C" {

int mi_add2_rmsnorm_scalar(float* hidden, const float* a, const float* b, const int* rows, const float* gain1,
                           const float* gain2, void* out1, void* out2, int adtype, int n, int H, float eps,
                           cudaStream_t stream) {
    if (n <= 0 || H <= 0) return kOk;
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(add2_rmsnorm_scalar_kernel<AT>, dim3(n), dim3(256), 0, stream, hidden, a, b, rows, gain1,
                         gain2, (AT*)out1, (AT*)out2, H, eps));
    return finish_launch("add2_rmsnorm_scalar");
}

int mi_geglu_tanh(const void* gu, void* out, int adtype, int64_t T, int I, cudaStream_t stream) {
    const int64_t total = T * I;
    if (total <= 0) return kOk;
    if (adtype == kBF16 && I % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int64_t total_vec = total / 8;
        int64_t vblocks = (total_vec + 255) / 256;
        if (vblocks > 148 * 16) vblocks = 148 * 16;
        launch_dependent(geglu_tanh_bf16x8_kernel, dim3((int)vblocks), dim3(256), 0, stream, (const uint4*)gu,
                         (uint4*)out, total_vec, I / 8);
        return finish_launch("geglu_tanh");
    }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(geglu_tanh_kernel<AT>, dim3((int)blocks), dim3(256), 0, stream, (const AT*)gu, (AT*)out,
                         total, I));
    return finish_launch("geglu_tanh");
}

int mi_clamped_glu(const float* gu, void* out, int adtype, int64_t T, int I, float limit, float slope,
                   cudaStream_t stream) {
    const int64_t total = T * I;
    if (total <= 0) return kOk;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(clamped_glu_kernel<AT>, dim3((int)blocks), dim3(256), 0, stream, gu, (AT*)out, total, I,
                         limit, slope));
    return finish_launch("clamped_glu");
}

int mi_concat_cast(const float* hidden, const float* a, const float* b, const float* other, void* out, int adtype,
                   int T, int H, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return kOk;
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(concat_cast_kernel<AT>, dim3(T), dim3(256), 0, stream, hidden, a, b, other, (AT*)out, H));
    return finish_launch("concat_cast");
}

int mi_rows_plus_vec(float* hidden, const float* y, const void* vec, int wdtype, int T, int H, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return kOk;
    MI_DISPATCH_1(wdtype, WT,
        launch_dependent(rows_plus_vec_kernel<WT>, dim3(T), dim3(256), 0, stream, hidden, y, (const WT*)vec, H));
    return finish_launch("rows_plus_vec");
}

int mi_group_rmsnorm(const float* x, const int* rows, const void* w, int wdtype, void* out, int odtype, int n, int H,
                     int groups, float eps, cudaStream_t stream) {
    if (n <= 0 || H <= 0) return kOk;
    if (groups < 1 || H % groups || groups > 65535) {
        set_last_error("group norm: %d columns do not split into %d groups", H, groups);
        return kBadShape;
    }
    const int gs = H / groups;
    const bool vec = gs % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int work = vec ? gs / 4 : gs;
    int threads = 32;
    while (threads < work && threads < 256) threads *= 2;
    MI_DISPATCH_2(odtype, OT, wdtype, WT,
        launch_dependent(group_rmsnorm_kernel<OT, WT>, dim3(n, groups), dim3(threads), 0, stream, x, rows,
                         (const WT*)w, (OT*)out, H, gs, eps, vec));
    return finish_launch("group_rmsnorm");
}

static int out_norm_add_groups(float* hidden, const float* y, const float* rows, const int* index, const float* wk,
                               const float* extra, const float* scale, int K, const void* w, int wdtype, void* x_out,
                               int adtype, int T, int H, float eps, float mult, int groups, cudaStream_t stream);

int mi_out_norm_add(float* hidden, const float* y, const float* rows, const int* index, const float* wk,
                    const float* extra, const float* scale, int K, const void* w, int wdtype, void* x_out, int adtype,
                    int T, int H, float eps, float mult, cudaStream_t stream) {
    return out_norm_add_groups(hidden, y, rows, index, wk, extra, scale, K, w, wdtype, x_out, adtype, T, H, eps, mult,
                               1, stream);
}

// the same with the root mean square of each of `groups` equal consecutive parts of the row by itself
int mi_out_norm_add_groups(float* hidden, const float* y, const float* rows, const int* index, const float* wk,
                           const float* extra, const float* scale, int K, const void* w, int wdtype, void* x_out,
                           int adtype, int T, int H, float eps, float mult, int groups, cudaStream_t stream) {
    return out_norm_add_groups(hidden, y, rows, index, wk, extra, scale, K, w, wdtype, x_out, adtype, T, H, eps, mult,
                               groups, stream);
}

static int out_norm_add_groups(float* hidden, const float* y, const float* rows, const int* index, const float* wk,
                               const float* extra, const float* scale, int K, const void* w, int wdtype, void* x_out,
                               int adtype, int T, int H, float eps, float mult, int groups, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return kOk;
    if (groups < 1 || H % groups || groups > 65535) {
        set_last_error("out_norm_add: %d columns do not split into %d groups", H, groups);
        return kBadShape;
    }
    const int gs = H / groups;
    if (!y && (!rows || K < 1)) { set_last_error("out_norm_add: neither a tensor nor rows to add"); return kBadShape; }
    if ((extra == nullptr) != (scale == nullptr)) {
        set_last_error("out_norm_add: the extra term and its scale come together");
        return kBadShape;
    }
    const RowSum s{y, rows, index, wk, extra, scale, K};
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(y) |
                           reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(extra) |
                           reinterpret_cast<uintptr_t>(x_out);
    if (gs % 4 == 0 && gs <= 8192 && (ptrs & 15) == 0) {
#define MI_OUT_NORM_VEC(VPT)                                                                                         \
    MI_DISPATCH_2(adtype, AT, wdtype, WT,                                                                            \
        launch_dependent(out_norm_add_vec_kernel<AT, WT, VPT>, dim3(T, groups), dim3(vthreads), 0, stream, hidden, s, \
                         (const WT*)w, (AT*)x_out, H, eps, mult, gs))
        // a group narrower than 1024 columns takes a smaller block (with one group the block is as it always was,
        // and with it the order of the sum of squares)
        int vthreads = 256;
        if (groups > 1) while (vthreads > 32 && vthreads * 2 >= gs) vthreads /= 2;
        if (gs <= 1024) { MI_OUT_NORM_VEC(1); }
        else if (gs <= 2048) { MI_OUT_NORM_VEC(2); }
        else if (gs <= 4096) { MI_OUT_NORM_VEC(4); }
        else { MI_OUT_NORM_VEC(8); }
#undef MI_OUT_NORM_VEC
        return finish_launch("out_norm_add");
    }
    const size_t smem = gs <= 8192 ? sizeof(float) * gs : 0;
    MI_DISPATCH_2(adtype, AT, wdtype, WT,
        launch_dependent(out_norm_add_kernel<AT, WT>, dim3(T, groups), dim3(256), smem, stream, hidden, s, (const WT*)w,
                         (AT*)x_out, H, eps, mult, gs));
    return finish_launch("out_norm_add");
}

int mi_softcap_rows(float* z, int64_t total, float cap, cudaStream_t stream) {
    if (total <= 0) return kOk;
    if (!(cap > 0.f)) { set_last_error("softcap_rows: the cap must be positive"); return kBadShape; }
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    launch_dependent(softcap_rows_kernel, dim3((int)blocks), dim3(256), 0, stream, z, total, cap);
    return finish_launch("softcap_rows");
}

int mi_cast_rows(const float* x, void* out, int adtype, int64_t total, cudaStream_t stream) {
    if (total <= 0) return kOk;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(cast_rows_kernel<AT>, dim3((int)blocks), dim3(256), 0, stream, x, (AT*)out, total));
    return finish_launch("cast_rows");
}

}  // extern "C"
