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
    if (threadIdx.x < N * N) c.mix[threadIdx.x] = mix ? mix[threadIdx.x] : 0.0f;
    if (threadIdx.x < N) {
        c.out[threadIdx.x] = outw ? outw[threadIdx.x] : 0.0f;
        c.in[threadIdx.x] = inw ? inw[threadIdx.x] : 1.0f;
    }
    pdl_wait();
    __syncthreads();
    const int r = blockIdx.x;
    const size_t t = rows ? (size_t)rows[r] : (size_t)r;
    float* base = lanes + t * d;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d; i += LANE_THREADS) {
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
        if (z_out) for (int i = threadIdx.x; i < d; i += LANE_THREADS) z_out[(size_t)r * d + i] = z_s[i];
        return;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += LANE_THREADS) {
        const float z = z_s[i];
        h[(size_t)r * d + i] = from_float<TH>(z * inv * g[i]);
        if (z_out) z_out[(size_t)r * d + i] = z;
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
#define BG_LANE_LAUNCH(N)                                                                                              \
    do {                                                                                                               \
        auto kern = lane_step_kernel<TY, TH, N>;                                                                       \
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch(kern, dim3(n_rows), dim3(LANE_THREADS), smem, stream, lanes, (size_t)lane_stride, (const TY*)y, parts,  \
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
