// A residual kept in several lanes (hyper-connections): L_1 .. L_n, float [n][T][d].
//
// A sublayer with constants (r [n], M [n][n], w [n]) reads z = sum_a r_a L_a, and its result y replaces all lanes at
// once: L_b <- sum_a M[a][b] L_a + w_b y.  The write of one sublayer and the read of the next are one pass over the
// lanes, fused with the RMS norm that stands in front of the next sublayer:
//
//   lane_step   per row t: (1) if a result is owed, the lanes are rewritten from it (y as it is, in either type, or the
//               sum of a split-K product's float partial sums, added in index order); (2) z = sum_a r_a L_a of the new
//               lanes; (3) h = z / sqrt(mean(z^2) + eps) * g in the compute type and/or z itself as float.
//
// One block per row; a thread keeps its columns' lanes in registers between (1) and (2), z goes through shared memory
// between the sum of squares and the scaling.  Everything is float.  A row's arithmetic does not depend on the step's
// other rows.
#include "common.cuh"

namespace bg {

constexpr int LANES_MAX = 8;
constexpr int LANE_THREADS = 256;

struct LaneConsts {
    float mix[LANES_MAX * LANES_MAX];   // [from][to]
    float out[LANES_MAX];
    float in[LANES_MAX];
};

template <typename TY, typename TH, int N>
__global__ void __launch_bounds__(LANE_THREADS)
lane_step_kernel(float* __restrict__ lanes, size_t lane_stride, const TY* __restrict__ y, int parts, size_t part_stride,
                 const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                 const float* __restrict__ g, float eps, TH* __restrict__ h, float* __restrict__ z_out,
                 const int* __restrict__ rows, int d) {
    extern __shared__ float z_s[];                         // [d]
    __shared__ float red[32];
    __shared__ LaneConsts c;
    pdl_launch();
    for (int k = threadIdx.x; k < N * N; k += blockDim.x) c.mix[k] = mix ? mix[k] : 0.0f;
    for (int k = threadIdx.x; k < N; k += blockDim.x) {
        c.out[k] = outw ? outw[k] : 0.0f;
        c.in[k] = inw ? inw[k] : 1.0f;
    }
    pdl_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    float* base = lanes + t * d;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float x[N];
#pragma unroll
        for (int a = 0; a < N; ++a) x[a] = base[(size_t)a * lane_stride + i];
        if (y) {
            const float yv = sum_parts(y + t * d + i, parts, part_stride);
            float nx[N];
#pragma unroll
            for (int b = 0; b < N; ++b) {
                float acc = 0.0f;
#pragma unroll
                for (int a = 0; a < N; ++a) acc = fmaf(c.mix[a * N + b], x[a], acc);
                nx[b] = fmaf(c.out[b], yv, acc);
            }
#pragma unroll
            for (int b = 0; b < N; ++b) {
                x[b] = nx[b];
                if (!rows) base[(size_t)b * lane_stride + i] = nx[b];     // (gathered rows are read, not rewritten)
            }
        }
        float z = 0.0f;
#pragma unroll
        for (int a = 0; a < N; ++a) z = fmaf(c.in[a], x[a], z);
        z_s[i] = z;
        ss = fmaf(z, z, ss);
    }
    if (!h) {
        if (z_out) for (int i = threadIdx.x; i < d; i += blockDim.x) z_out[(size_t)r * d + i] = z_s[i];
        return;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float z = z_s[i];
        h[(size_t)r * d + i] = from_float<TH>(z * inv * g[i]);
        if (z_out) z_out[(size_t)r * d + i] = z;
    }
}

// Four columns of an owed result as floats: the sum of a product's float partial sums, or one row in bfloat16.
__device__ __forceinline__ float4 owed4(const float* y, size_t at, int parts, size_t part_stride) {
    return sum_parts4(reinterpret_cast<const float4*>(y + at), parts, part_stride / 4);
}
__device__ __forceinline__ float4 owed4(const __nv_bfloat16* y, size_t at, int, size_t) {
    const uint2 raw = *reinterpret_cast<const uint2*>(y + at);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

// The same pass, four columns a thread (d a multiple of 4, rows on 16-byte boundaries): all of a thread's loads (its
// columns of every lane and of every partial sum) go out before the first sum, so a row costs one trip to memory, the
// exchange of the sums of squares, and the stores.  The read z stays in shared memory between the two.
template <typename TY, typename TH, int N>
__global__ void __launch_bounds__(512)
lane_step_vec4_kernel(float* __restrict__ lanes, size_t lane_stride, const TY* __restrict__ y, int parts, size_t part_stride,
                      const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
                      const float* __restrict__ g, float eps, TH* __restrict__ h, float* __restrict__ z_out,
                      const int* __restrict__ rows, int d) {
    extern __shared__ float4 z4_s[];                       // [d / 4]
    __shared__ float red[32];
    __shared__ LaneConsts c;
    pdl_launch();
    for (int k = threadIdx.x; k < N * N; k += blockDim.x) c.mix[k] = mix ? mix[k] : 0.0f;
    for (int k = threadIdx.x; k < N; k += blockDim.x) {
        c.out[k] = outw ? outw[k] : 0.0f;
        c.in[k] = inw ? inw[k] : 1.0f;
    }
    pdl_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    float* base = lanes + t * d;
    float ss = 0.0f;
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 x[N];
#pragma unroll
        for (int a = 0; a < N; ++a) x[a] = *reinterpret_cast<const float4*>(base + (size_t)a * lane_stride + i);
        if (y) {
            const float4 yv = owed4(y, t * d + i, parts, part_stride);
            float4 nx[N];
#pragma unroll
            for (int b = 0; b < N; ++b) {
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int a = 0; a < N; ++a) {
                    const float m = c.mix[a * N + b];
                    acc.x = fmaf(m, x[a].x, acc.x); acc.y = fmaf(m, x[a].y, acc.y);
                    acc.z = fmaf(m, x[a].z, acc.z); acc.w = fmaf(m, x[a].w, acc.w);
                }
                const float o = c.out[b];
                nx[b] = make_float4(fmaf(o, yv.x, acc.x), fmaf(o, yv.y, acc.y), fmaf(o, yv.z, acc.z), fmaf(o, yv.w, acc.w));
            }
#pragma unroll
            for (int b = 0; b < N; ++b) {
                x[b] = nx[b];
                if (!rows) *reinterpret_cast<float4*>(base + (size_t)b * lane_stride + i) = nx[b];
            }
        }
        float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int a = 0; a < N; ++a) {
            const float w = c.in[a];
            z.x = fmaf(w, x[a].x, z.x); z.y = fmaf(w, x[a].y, z.y); z.z = fmaf(w, x[a].z, z.z); z.w = fmaf(w, x[a].w, z.w);
        }
        z4_s[i >> 2] = z;
        ss = fmaf(z.x, z.x, ss); ss = fmaf(z.y, z.y, ss); ss = fmaf(z.z, z.z, ss); ss = fmaf(z.w, z.w, ss);
        if (z_out) *reinterpret_cast<float4*>(z_out + (size_t)r * d + i) = z;
    }
    if (!h) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        const float4 z = z4_s[i >> 2];
        const float4 w = *reinterpret_cast<const float4*>(g + i);
        store4(h + (size_t)r * d + i, make_float4(z.x * inv * w.x, z.y * inv * w.y, z.z * inv * w.z, z.w * inv * w.w));
    }
}

// lanes[a][t][:] = x[t][:] for every lane a: the start of a model that keeps its residual in lanes.
__global__ void lane_fill_kernel(const float* __restrict__ x, float* __restrict__ lanes, size_t n, int count) {
    pdl_launch();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    for (int a = 0; a < count; ++a) lanes[(size_t)a * n + i] = v;
}

}  // namespace bg

using namespace bg;

// lanes float [n][T][d] (lane_stride elements between lanes).  y (may be null): the owed result [T][d] of y_dtype, or
// float partial sums [parts][T][d]; then mix [n][n] and outw [n] rewrite the lanes.  inw [n] (null: ones) weighs the
// read.  g float [d] with h (of h_dtype, [n_rows][d]): the normed read; z_out float [n_rows][d]: the read itself.  rows
// (may be null): the rows to read, in which case nothing is written back to the lanes.
extern "C" int bg_lane_step(float* lanes, int n, long long lane_stride, const void* y, int y_dtype, int parts,
                            long long part_stride, const float* mix, const float* outw, const float* inw, const float* g,
                            float eps, void* h, int h_dtype, float* z_out, const int* rows, int n_rows, int d,
                            cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (n < 1 || n > LANES_MAX || d <= 0) return BG_ERR_SHAPE;
    if (y && (!mix || !outw)) return BG_ERR_SHAPE;
    if (h && !g) return BG_ERR_SHAPE;
    if (!y) { y_dtype = BG_DTYPE_F32; parts = 0; }
    if (y_dtype != BG_DTYPE_F32 && parts != 1) return BG_ERR_DTYPE;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_UNSUPPORTED;
    const bool vec = d % 4 == 0 && lane_stride % 4 == 0 && part_stride % 4 == 0 && (uintptr_t)lanes % 16 == 0 &&
                     (uintptr_t)y % 16 == 0 && (uintptr_t)g % 16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)z_out % 16 == 0;
    // a thread per four columns where the row allows it: one trip to memory a row (steps of few rows are bound by that trip)
    const int threads = vec ? ((d / 4 + 31) / 32 * 32 > 512 ? 512 : (d / 4 + 31) / 32 * 32) : LANE_THREADS;
#define BG_LANE_LAUNCH(N)                                                                                              \
    do {                                                                                                               \
        auto kern = vec ? lane_step_vec4_kernel<TY, TH, N> : lane_step_kernel<TY, TH, N>;                              \
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch(kern, dim3(n_rows), dim3(threads), smem, stream, lanes, (size_t)lane_stride, (const TY*)y, parts,       \
               (size_t)part_stride, mix, outw, inw, g, eps, (TH*)h, z_out, rows, d);                                   \
    } while (0)
    BG_DISPATCH_DTYPE(y_dtype, TY, BG_DISPATCH_DTYPE(h_dtype, TH, {
        switch (n) {
            case 1: BG_LANE_LAUNCH(1); break;
            case 2: BG_LANE_LAUNCH(2); break;
            case 3: BG_LANE_LAUNCH(3); break;
            case 4: BG_LANE_LAUNCH(4); break;
            case 5: BG_LANE_LAUNCH(5); break;
            case 6: BG_LANE_LAUNCH(6); break;
            case 7: BG_LANE_LAUNCH(7); break;
            default: BG_LANE_LAUNCH(8); break;
        }
    }));
#undef BG_LANE_LAUNCH
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_lane_fill(const float* x, float* lanes, long long n, int count, cudaStream_t stream) {
    if (n <= 0 || count <= 0) return BG_OK;
    launch(lane_fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, lanes, (size_t)n, count);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
