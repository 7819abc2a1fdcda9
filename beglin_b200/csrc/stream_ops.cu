// Small kernels around the residual stream and the activations that the Qwen2 parts do not have:
// the centred norm (LayerNorm without a shift) with the residual add in front of it, the depth-weighted average of the layer results,
// the xIELU activation, an RMS norm over a slice of a product's rows, and the per-head output gate.
// All statistics and sums are float; every row's sums run in an order fixed by the sizes alone.
#include "common.cuh"

namespace bg {

// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] + sum_p delta[p][s];  if update: x[s] = v;
//   out[r] = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w
// One block per row; the row is held in shared memory between the passes (sum, squared deviations, output).
template <typename TD, typename TW, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                                     const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                     const int* __restrict__ rows, int d, int update) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) v += sum_parts(delta + (size_t)s * d + i, parts, part_stride);
        row_buf[i] = v;
        if (update) xr[i] = v;
        sum += v;
    }
    sum = block_sum(sum, red);
    const float mean = sum / (float)d;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float dv = row_buf[i] - mean;
        sq += dv * dv;
    }
    sq = block_sum(sq, red);
    const float inv = 1.0f / sqrtf(sq / (float)d + eps);
    TO* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        o[i] = from_float<TO>((row_buf[i] - mean) * inv * to_float(w[i]));
}

// The same for a width that is a multiple of 8 with rows on 16-byte boundaries: a thread holds up to ITER runs of eight
// features in registers, all its loads (the row and every partial sum) on their way together, so a row is one round
// trip to memory instead of one per 256 features.  256 threads; d <= 2048 ITER.
template <typename TD, typename TW, typename TO, int ITER>
__global__ void __launch_bounds__(256)
add_layernorm_vec8_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                          const TW* __restrict__ w, float eps, TO* __restrict__ out, const int* __restrict__ rows, int d,
                          int update) {
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const int s = rows ? rows[r] : r;
    float* xr = x + (size_t)s * d;
    const int d8 = d / 8;
    float v[ITER][8];
    float sum = 0.0f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int c = threadIdx.x + it * 256;
        if (c < d8) {
            load8(xr + c * 8, v[it]);
            for (int pp = 0; pp < parts; ++pp) {
                float dv[8];
                load8(delta + (size_t)pp * part_stride + (size_t)s * d + c * 8, dv);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[it][k] += dv[k];
            }
            if (update) store8(xr + c * 8, v[it]);
#pragma unroll
            for (int k = 0; k < 8; ++k) sum += v[it][k];
        }
    }
    sum = block_sum(sum, red);
    const float mean = sum / (float)d;
    float sq = 0.0f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int c = threadIdx.x + it * 256;
        if (c < d8) {
#pragma unroll
            for (int k = 0; k < 8; ++k) { const float dv = v[it][k] - mean; sq += dv * dv; }
        }
    }
    sq = block_sum(sq, red);
    const float inv = 1.0f / sqrtf(sq / (float)d + eps);
    TO* o = out + (size_t)r * d;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int c = threadIdx.x + it * 256;
        if (c < d8) {
            float wv[8], ov[8];
            load8(w + c * 8, wv);
#pragma unroll
            for (int k = 0; k < 8; ++k) ov[k] = (v[it][k] - mean) * inv * wv[k];
            store8(o + c * 8, ov);
        }
    }
}

// The depth-weighted average behind a layer.  With v = x + sum_p delta[p] (the layer's result):
//   history[terms - 1] = v;   x = sum_{j < terms} w[j] * history[j], added in the order of j.
// history is [slots][n] with hist_stride elements between slots; slots 0 .. terms-2 were written earlier.
template <typename TD, typename TW>
__global__ void depth_mix_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                                 float* __restrict__ history, size_t hist_stride, const TW* __restrict__ w, int terms,
                                 size_t n) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (delta) v += sum_parts(delta + i, parts, part_stride);
    history[(size_t)(terms - 1) * hist_stride + i] = v;
    float acc = 0.0f;
    for (int j = 0; j + 1 < terms; ++j) acc = fmaf(to_float(w[j]), history[(size_t)j * hist_stride + i], acc);
    x[i] = fmaf(to_float(w[terms - 1]), v, acc);
}

// The same, eight values a thread with 16-byte accesses (n a multiple of 8, everything on 16-byte boundaries): the
// loads of all terms are independent of one another.
template <typename TD, typename TW>
__global__ void depth_mix_vec8_kernel(float* __restrict__ x, const TD* __restrict__ delta, int parts, size_t part_stride,
                                      float* __restrict__ history, size_t hist_stride, const TW* __restrict__ w, int terms,
                                      size_t n8) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    float v[8];
    load8(x + i * 8, v);
    for (int pp = 0; pp < parts; ++pp) {
        float dv[8];
        load8(delta + (size_t)pp * part_stride + i * 8, dv);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] += dv[k];
    }
    store8(history + (size_t)(terms - 1) * hist_stride + i * 8, v);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    for (int j = 0; j + 1 < terms; ++j) {
        const float wj = to_float(w[j]);
        float hj[8];
        load8(history + (size_t)j * hist_stride + i * 8, hj);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = fmaf(wj, hj[k], acc[k]);
    }
    const float wl = to_float(w[terms - 1]);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = fmaf(wl, v[k], acc[k]);
    store8(x + i * 8, acc);
}

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// out = xIELU(z), z = in or the sum of its partial sums.  With a_pos = softplus(act[0]) and
// a_neg = 1/2 + softplus(act[1]):   z > 0:  z (a_pos z + 1/2);    else:  a_neg (expm1(z) - z) + z/2
__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
    return z > 0.0f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
}

template <typename TI, typename TW, typename TO>
__global__ void xielu_kernel(const TI* __restrict__ in, int parts, size_t part_stride, const TW* __restrict__ act,
                             TO* __restrict__ out, size_t n) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float ap = softplus_f(to_float(act[0]));
    const float an = 0.5f + softplus_f(to_float(act[1]));
    const float z = parts > 1 ? sum_parts(in + i, parts, part_stride) : to_float(in[i]);
    out[i] = from_float<TO>(xielu_f(z, ap, an));
}

// The same for one complete input whose size is a multiple of 8 and whose rows lie on 16-byte boundaries: eight
// values a thread, 16-byte loads and stores.
template <typename TI, typename TW, typename TO>
__global__ void xielu_vec8_kernel(const TI* __restrict__ in, const TW* __restrict__ act, TO* __restrict__ out, size_t n8) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float ap = softplus_f(to_float(act[0]));
    const float an = 0.5f + softplus_f(to_float(act[1]));
    float v[8];
    load8(in + i * 8, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = xielu_f(v[k], ap, an);
    store8(out + i * 8, v);
}

// out[r, 0..n) = s * rsqrt(mean(s^2) + eps) * w, s = src[r, col0 .. col0 + n): the RMS norm of a slice of
// the rows of a product.  One block per row.
template <typename TI, typename TW, typename TO>
__global__ void rmsnorm_slice_kernel(const TI* __restrict__ src, int src_stride, int col0, int n,
                                     const TW* __restrict__ w, float eps, TO* __restrict__ out, int out_stride) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const TI* s = src + (size_t)r * src_stride + col0;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = to_float(s[i]);
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    TO* o = out + (size_t)r * out_stride;
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_float<TO>(row_buf[i] * inv * to_float(w[i]));
}

// out[t, h * vd + j] = src[h][t][j] * sigmoid(gate[t, gate_col0 + h]): head-major results put row by row,
// each head scaled by its gate (without `gate`: put row by row as they are).
template <typename TI, typename TG, typename TO>
__global__ void gate_heads_kernel(const TI* __restrict__ src, size_t src_head_stride, int src_row_stride,
                                  const TG* __restrict__ gate, int gate_stride, int gate_col0, TO* __restrict__ out,
                                  int T, int H, int vd) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = (size_t)T * H * vd;
    if (i >= n) return;
    const int j = (int)(i % vd);
    const int h = (int)((i / vd) % H);
    const int t = (int)(i / ((size_t)vd * H));
    const float s = gate ? 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + gate_col0 + h]))) : 1.0f;
    out[i] = from_float<TO>(to_float(src[(size_t)h * src_head_stride + (size_t)t * src_row_stride + j]) * s);
}

// The same, eight features a thread (vd a multiple of 8, rows on 16-byte boundaries).
template <typename TI, typename TG, typename TO>
__global__ void gate_heads_vec8_kernel(const TI* __restrict__ src, size_t src_head_stride, int src_row_stride,
                                       const TG* __restrict__ gate, int gate_stride, int gate_col0, TO* __restrict__ out,
                                       int T, int H, int vd) {
    pdl_launch();
    pdl_wait();
    const int v8 = vd / 8;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = (size_t)T * H * v8;
    if (i >= n) return;
    const int j = (int)(i % v8);
    const int h = (int)((i / v8) % H);
    const int t = (int)(i / ((size_t)v8 * H));
    const float sg = gate ? 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_stride + gate_col0 + h]))) : 1.0f;
    float v[8];
    load8(src + (size_t)h * src_head_stride + (size_t)t * src_row_stride + j * 8, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= sg;
    store8(out + ((size_t)t * H + h) * vd + j * 8, v);
}

}  // namespace bg

using namespace bg;

template <typename TD, typename TW>
static int add_layernorm_out(float* x, const void* delta, int parts, size_t part_stride, const void* w, float eps, void* out,
                             int out_dtype, const int* rows, int n_rows, int d, int update, cudaStream_t stream) {
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    const bool vec = (d % 8 == 0) && (part_stride % 8 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)delta % 16 == 0) &&
                     ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0) && d <= 8192;
    if (vec) {
        const int iter = (d / 8 + 255) / 256;
        BG_DISPATCH_DTYPE(out_dtype, TO, {
            if (iter <= 1) launch(add_layernorm_vec8_kernel<TD, TW, TO, 1>, dim3(n_rows), dim3(256), 0, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
            else if (iter <= 2) launch(add_layernorm_vec8_kernel<TD, TW, TO, 2>, dim3(n_rows), dim3(256), 0, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
            else launch(add_layernorm_vec8_kernel<TD, TW, TO, 4>, dim3(n_rows), dim3(256), 0, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps, (TO*)out, rows, d, update);
        });
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    BG_DISPATCH_DTYPE(out_dtype, TO, {
        auto kern = add_layernorm_kernel<TD, TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kern, dim3(n_rows), dim3(256), smem, stream, x, (const TD*)delta, parts, part_stride, (const TW*)w, eps,
               (TO*)out, rows, d, update);
    });
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// The arguments of bg_add_rmsnorm, for the centred norm (scale vector, no shift).
extern "C" int bg_add_layernorm(float* x, const void* delta, int delta_dtype, int parts, long long part_stride,
                                const void* w, int w_dtype, float eps, void* out, int out_dtype, const int* rows,
                                int n_rows, int d, int update, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (!delta) { delta_dtype = BG_DTYPE_F32; parts = 0; }
    BG_DISPATCH_DTYPE(delta_dtype, TD, BG_DISPATCH_DTYPE(w_dtype, TW,
        return (add_layernorm_out<TD, TW>(x, delta, parts, (size_t)part_stride, w, eps, out, out_dtype, rows, n_rows, d,
                                          update, stream))));
    return BG_OK;
}

extern "C" int bg_depth_mix(float* x, const void* delta, int delta_dtype, int parts, long long part_stride, float* history,
                            long long hist_stride, const void* w, int w_dtype, int terms, long long n, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    if (terms < 1) return BG_ERR_SHAPE;
    if (!delta) { delta_dtype = BG_DTYPE_F32; parts = 0; }
    if (n % 8 == 0 && hist_stride % 8 == 0 && part_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)delta % 16 == 0 &&
        (uintptr_t)history % 16 == 0) {
        const size_t n8 = (size_t)n / 8;
        BG_DISPATCH_DTYPE(delta_dtype, TD, BG_DISPATCH_DTYPE(w_dtype, TW,
            launch(depth_mix_vec8_kernel<TD, TW>, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, x, (const TD*)delta, parts,
                   (size_t)part_stride, history, (size_t)hist_stride, (const TW*)w, terms, n8)));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(delta_dtype, TD, BG_DISPATCH_DTYPE(w_dtype, TW,
        launch(depth_mix_kernel<TD, TW>, dim3(blocks), dim3(256), 0, stream, x, (const TD*)delta, parts, (size_t)part_stride,
               history, (size_t)hist_stride, (const TW*)w, terms, (size_t)n)));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_xielu(const void* in, int in_dtype, int parts, long long part_stride, const void* act, int act_dtype,
                        void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return BG_OK;
    if (parts > 1 && in_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;
    if (parts <= 1 && n % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t n8 = (size_t)n / 8;
        const unsigned blocks8 = (unsigned)((n8 + 255) / 256);
        BG_DISPATCH_DTYPE(in_dtype, TI, BG_DISPATCH_DTYPE(act_dtype, TW, BG_DISPATCH_DTYPE(out_dtype, TO,
            launch(xielu_vec8_kernel<TI, TW, TO>, dim3(blocks8), dim3(256), 0, stream, (const TI*)in, (const TW*)act, (TO*)out, n8))));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(in_dtype, TI, BG_DISPATCH_DTYPE(act_dtype, TW, BG_DISPATCH_DTYPE(out_dtype, TO,
        launch(xielu_kernel<TI, TW, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)in, parts, (size_t)part_stride,
               (const TW*)act, (TO*)out, (size_t)n))));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_rmsnorm_slice(const void* src, int src_dtype, int src_stride, int col0, int n, const void* w, int w_dtype,
                                float eps, void* out, int out_dtype, int out_stride, int rows, cudaStream_t stream) {
    if (rows <= 0) return BG_OK;
    if (n <= 0) return BG_ERR_SHAPE;
    const size_t smem = (size_t)n * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    const int threads = n >= 256 ? 256 : (n + 31) / 32 * 32;
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(out_dtype, TO, {
        auto kern = rmsnorm_slice_kernel<TI, TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kern, dim3(rows), dim3(threads), smem, stream, (const TI*)src, src_stride, col0, n, (const TW*)w, eps, (TO*)out,
               out_stride);
    })));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_gate_heads(const void* src, int src_dtype, long long src_head_stride, int src_row_stride, const void* gate,
                             int gate_dtype, int gate_stride, int gate_col0, void* out, int out_dtype, int T, int H, int vd,
                             cudaStream_t stream) {
    const long long n = (long long)T * H * vd;
    if (n <= 0) return BG_OK;
    if (vd % 8 == 0 && src_head_stride % 8 == 0 && src_row_stride % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t n8 = (size_t)n / 8;
        BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(gate_dtype, TG, BG_DISPATCH_DTYPE(out_dtype, TO,
            launch(gate_heads_vec8_kernel<TI, TG, TO>, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (const TI*)src,
                   (size_t)src_head_stride, src_row_stride, (const TG*)gate, gate_stride, gate_col0, (TO*)out, T, H, vd))));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(gate_dtype, TG, BG_DISPATCH_DTYPE(out_dtype, TO,
        launch(gate_heads_kernel<TI, TG, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)src, (size_t)src_head_stride,
               src_row_stride, (const TG*)gate, gate_stride, gate_col0, (TO*)out, T, H, vd))));
    BG_LAUNCH_CHECK();
    return BG_OK;
}
