// The Mamba-2 recurrence for a ragged step: every request brings a run of consecutive tokens (a prompt
// portion or one decoded token) and owns one slot of fixed state, float32:
//   slot = [ S: heads x P x N | conv: (taps - 1) x channels ]
// S is the state of the recurrence, conv the last taps-1 inputs of the causal convolution (oldest first).
// A slot is zero when its request starts, so a convolution that reaches back beyond a sequence's first
// token finds zeros there.  Four kernels: the convolution with SiLU, the update of its state, the scan, and the gate
// with the grouped RMS norm.  Everything that enters the recurrence is float: step sizes, decays, B, C, x.
//
// Requests are given as a list of (request, first row, number of rows), one entry per request of the step.
#include "common.cuh"

namespace bg {

__device__ __forceinline__ float softplus32(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu32(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid32(float z) { return 1.0f / (1.0f + expf(-z)); }

// out[t, c] = silu(b[c] + sum_j w[c, j] * in(t - (taps-1-j), c)), in(.) taken from the step's rows of the same
// request or, further back, from the slot's conv state.  src row = [.. | channels from col0 | ..].  `src_bias` [channels]
// (may be null) is added to every input taken from the step's rows, and the state keeps inputs with it: what lies before a
// request's start stays zero.
template <typename TI, typename TW>
__global__ void conv_silu_kernel(const TI* __restrict__ src, int src_stride, int col0, int channels, int taps,
                                 const TW* __restrict__ w, const TW* __restrict__ b, const float* __restrict__ state,
                                 size_t slot_stride, size_t conv_off, const int* __restrict__ slots,
                                 const int* __restrict__ row_req, const int* __restrict__ reqs, float* __restrict__ out,
                                 int act, const float* __restrict__ src_bias) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= channels) return;
    const int req = row_req[t];
    const int row0 = reqs[req * 3 + 1];
    const int j = t - row0;                                   // rows of this request before this one in the step
    const float* st = state + (size_t)slots[req] * slot_stride + conv_off;
    float acc = to_float(b[c]);
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;
        float v;
        if (back <= j) v = to_float(src[(size_t)(t - back) * src_stride + col0 + c]) + (src_bias ? src_bias[c] : 0.0f);
        else v = st[(size_t)(taps - 1 - (back - j)) * channels + c];
        acc = fmaf(to_float(w[(size_t)c * taps + k]), v, acc);
    }
    out[(size_t)t * channels + c] = act ? silu32(acc) : acc;
}

// The slot's conv state after the step: the last taps-1 inputs of (old state, the step's n rows).
template <typename TI>
__global__ void conv_state_kernel(const TI* __restrict__ src, int src_stride, int col0, int channels, int taps,
                                  float* __restrict__ state, size_t slot_stride, size_t conv_off,
                                  const int* __restrict__ slots, const int* __restrict__ reqs, const float* __restrict__ src_bias) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int req = blockIdx.y;
    if (c >= channels) return;
    const int row0 = reqs[req * 3 + 1], n = reqs[req * 3 + 2];
    if (n <= 0) return;
    float* st = state + (size_t)slots[req] * slot_stride + conv_off;
    const int keep = taps - 1;
    for (int k = 0; k < keep; ++k) {                          // reads run ahead of writes: k + n > k
        const int idx = k + n;                                // index into (old state ++ new rows)
        const float v = idx < keep ? st[(size_t)idx * channels + c]
                                   : to_float(src[(size_t)(row0 + idx - keep) * src_stride + col0 + c]) + (src_bias ? src_bias[c] : 0.0f);
        st[(size_t)k * channels + c] = v;
    }
}

// The scan.  One CTA per (head, request, tile of PT columns p); thread (pl, ns) = tid / NS, tid % NS owns NPT values
// S[n][p0 + pl] in registers: for NPT >= 4 the n come in runs of four, n = ((k / 4) NS + ns) 4 + k % 4, so that a
// token's B and C reach a thread as 16-byte loads from shared memory without bank conflicts between the NS
// neighbours (B and C are padded with zeros up to NPT NS values); for fewer, n = ns + k NS.  Per token:
//   dt = softplus(dt_raw + dt_bias);  S = e^(-e^(A_log) dt) S + dt B x^T;  y = S^T C + D x.
// The tokens go through shared memory in chunks of SCAN_CHUNK; the sum over n ends with shuffles among the NS
// neighbouring lanes of a p.  A token's arithmetic does not depend on where the step was cut.
constexpr int SCAN_CHUNK = 16;
constexpr int SCAN_THREADS = 512;

__device__ __forceinline__ void scan_cp_async4(float* smem_dst, const float* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem_src) : "memory");
}


// U tokens of the recurrence for one thread's states: the states move token by token, the U sums over n are then
// brought together side by side (their shuffles in flight together), and the U results stored.
template <int U, int NPT>
__device__ __forceinline__ void scan_tokens(float (&S)[NPT], const float* __restrict__ B_s, const float* __restrict__ C_s,
                                            const float* __restrict__ x_s, const float* __restrict__ dt_s,
                                            const float* __restrict__ da_s, float* __restrict__ y_s, int tt, int NP, int PT,
                                            int NS, int ns, int pl, bool live, float Dh) {
    float yv[U], xv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const float dt = dt_s[tt + u], dA = da_s[tt + u];
        xv[u] = live ? x_s[(tt + u) * PT + pl] : 0.0f;
        const float dtx = dt * xv[u];
        const float* Bt = B_s + (tt + u) * NP;
        const float* Ct = C_s + (tt + u) * NP;
        float y0 = 0.0f;
        if (NPT >= 4) {                                        // padded n hold B = C = 0: their S stays 0
            const float4* B4 = reinterpret_cast<const float4*>(Bt) + ns;
            const float4* C4 = reinterpret_cast<const float4*>(Ct) + ns;
            float y1 = 0.0f;
#pragma unroll
            for (int kq = 0; kq < NPT / 4; ++kq) {
                const float4 b = B4[kq * NS], c = C4[kq * NS];
                S[4 * kq + 0] = fmaf(dA, S[4 * kq + 0], dtx * b.x); y0 = fmaf(S[4 * kq + 0], c.x, y0);
                S[4 * kq + 1] = fmaf(dA, S[4 * kq + 1], dtx * b.y); y1 = fmaf(S[4 * kq + 1], c.y, y1);
                S[4 * kq + 2] = fmaf(dA, S[4 * kq + 2], dtx * b.z); y0 = fmaf(S[4 * kq + 2], c.z, y0);
                S[4 * kq + 3] = fmaf(dA, S[4 * kq + 3], dtx * b.w); y1 = fmaf(S[4 * kq + 3], c.w, y1);
            }
            y0 += y1;
        } else {
#pragma unroll
            for (int k = 0; k < NPT; ++k) {
                const int nn = ns + k * NS;
                S[k] = fmaf(dA, S[k], dtx * Bt[nn]);
                y0 = fmaf(S[k], Ct[nn], y0);
            }
        }
        yv[u] = y0;
    }
    for (int off = NS >> 1; off > 0; off >>= 1) {
#pragma unroll
        for (int u = 0; u < U; ++u) yv[u] += __shfl_xor_sync(0xffffffffu, yv[u], off);
    }
    if (live && ns == 0) {
#pragma unroll
        for (int u = 0; u < U; ++u) y_s[(tt + u) * PT + pl] = fmaf(Dh, xv[u], yv[u]);
    }
}

template <typename TI, typename TW, int NPT>
__global__ void __launch_bounds__(SCAN_THREADS)
ssm_scan_kernel(const float* __restrict__ xbc, int channels, const TI* __restrict__ src, int src_stride,
                int dt_col, const TW* __restrict__ dt_bias, const TW* __restrict__ A_log,
                const TW* __restrict__ Dw, float* __restrict__ state, size_t slot_stride,
                const int* __restrict__ slots, const int* __restrict__ reqs, float* __restrict__ y,
                int H, int P, int N, int G, int NS, int PT) {
    extern __shared__ float sm[];
    const int NP = NPT * NS;                      // N rounded up to what the threads hold
    // two buffers of [CHUNK][NP] B, [CHUNK][NP] C, [CHUNK][PT] x, [CHUNK] dt, [CHUNK] decay; one [CHUNK][PT] y
    const int buf_floats = SCAN_CHUNK * (2 * NP + PT + 2);
    float* y_s = sm + 2 * buf_floats;
    pdl_launch();
    pdl_wait();
    const int h = blockIdx.x, req = blockIdx.y, p0 = blockIdx.z * PT;
    const int row0 = reqs[req * 3 + 1], n = reqs[req * 3 + 2];
    if (n <= 0) return;
    const int tid = threadIdx.x;
    const int pl = tid / NS, ns = tid - pl * NS;
    const int pcol = p0 + pl;
    const int pt = min(PT, P - p0);               // columns of this tile
    const bool live = pl < pt;
    const int g = h / (H / G);
    const int inner = H * P;
    float* st = state + (size_t)slots[req] * slot_stride + (size_t)h * N * P;
    constexpr bool RUNS = NPT >= 4;               // runs of four n per thread
    float S[NPT];
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
        const int nn = RUNS ? ((k >> 2) * NS + ns) * 4 + (k & 3) : ns + k * NS;
        S[k] = (live && nn < N) ? st[(size_t)pcol * N + nn] : 0.0f;
    }
    const float a = expf(to_float(A_log[h]));
    const float bias = to_float(dt_bias[h]);
    const float Dh = to_float(Dw[h]);
    const float* Bsrc = xbc + inner + (size_t)g * N;
    const float* Csrc = xbc + inner + (size_t)G * N + (size_t)g * N;
    const float* xsrc = xbc + (size_t)h * P + p0;
    // the padding of B and C (n from N up to NP) is zero for good: it is written once, the copies never touch it
    for (int idx = tid; idx < 2 * SCAN_CHUNK * (NP - N); idx += blockDim.x) {
        const int bsel = idx / (SCAN_CHUNK * (NP - N)), r = idx - bsel * SCAN_CHUNK * (NP - N);
        const int tt = r / (NP - N), nn = N + (r - tt * (NP - N));
        float* bb = sm + bsel * buf_floats;
        bb[tt * NP + nn] = 0.0f;
        bb[SCAN_CHUNK * NP + tt * NP + nn] = 0.0f;
    }
    // a chunk's B, C and x on their way into a buffer: 4-byte asynchronous copies, so that they all are in flight at
    // once and the chunk after the one being computed is under way meanwhile
    auto issue = [&](int c0, int bsel) {
        float* bb = sm + bsel * buf_floats;
        const int tc = min(SCAN_CHUNK, n - c0);
        for (int tt = 0; tt < tc; ++tt) {
            const size_t row = (size_t)(row0 + c0 + tt) * channels;
            for (int nn = tid; nn < N; nn += blockDim.x) {
                scan_cp_async4(bb + tt * NP + nn, Bsrc + row + nn);
                scan_cp_async4(bb + SCAN_CHUNK * NP + tt * NP + nn, Csrc + row + nn);
            }
            for (int pp = tid; pp < pt; pp += blockDim.x) scan_cp_async4(bb + 2 * SCAN_CHUNK * NP + tt * PT + pp, xsrc + row + pp);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    auto raw_dt = [&](int c0) {
        return (tid < min(SCAN_CHUNK, n - c0)) ? to_float(src[(size_t)(row0 + c0 + tid) * src_stride + dt_col + h]) : 0.0f;
    };
    issue(0, 0);
    float dt_raw = raw_dt(0);
    int bsel = 0;
    for (int c0 = 0; c0 < n; c0 += SCAN_CHUNK, bsel ^= 1) {
        const int tc = min(SCAN_CHUNK, n - c0);
        float* bb = sm + bsel * buf_floats;
        const float* B_s = bb;
        const float* C_s = bb + SCAN_CHUNK * NP;
        const float* x_s = bb + 2 * SCAN_CHUNK * NP;
        float* dt_s = bb + 2 * SCAN_CHUNK * NP + SCAN_CHUNK * PT;
        float* da_s = dt_s + SCAN_CHUNK;
        if (tid < tc) {
            const float dt = softplus32(dt_raw + bias);
            dt_s[tid] = dt;
            da_s[tid] = expf(-a * dt);
        }
        const bool more = c0 + SCAN_CHUNK < n;
        if (more) {
            issue(c0 + SCAN_CHUNK, bsel ^ 1);
            dt_raw = raw_dt(c0 + SCAN_CHUNK);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        int tt = 0;
        for (; tt + 4 <= tc; tt += 4)
            scan_tokens<4, NPT>(S, B_s, C_s, x_s, dt_s, da_s, y_s, tt, NP, PT, NS, ns, pl, live, Dh);
        for (; tt < tc; ++tt)
            scan_tokens<1, NPT>(S, B_s, C_s, x_s, dt_s, da_s, y_s, tt, NP, PT, NS, ns, pl, live, Dh);
        __syncthreads();
        for (int idx = tid; idx < tc * pt; idx += blockDim.x) {
            const int tt = idx / pt, pp = idx - tt * pt;
            y[(size_t)(row0 + c0 + tt) * inner + (size_t)h * P + p0 + pp] = y_s[tt * PT + pp];
        }
    }
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
        const int nn = RUNS ? ((k >> 2) * NS + ns) * 4 + (k & 3) : ns + k * NS;
        if (live && nn < N) st[(size_t)pcol * N + nn] = S[k];
    }
}

// out[t, i] = v * rsqrt(mean over i's group of v^2 + eps) * w[i],  v = y[t, i] * silu(z[t, i]); the row is cut
// into `groups` equal parts, each with a root mean square of its own.  z = src[t, z_col + i].  One block per
// (row, group).  With `mode` 1 the gate stands behind the norm and is a sigmoid: v = y[t, i], and the normed value is
// multiplied by sigmoid(z[t, i]).
template <typename TI, typename TW, typename TO>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const TI* __restrict__ src, int src_stride, int z_col,
                                           const TW* __restrict__ w, float eps, TO* __restrict__ out, int inner, int groups, int mode) {
    extern __shared__ float row_buf[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y;
    const int gs = inner / groups;
    const int i0 = g * gs;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float z = to_float(src[(size_t)t * src_stride + z_col + i0 + i]);
        const float v = mode ? y[(size_t)t * inner + i0 + i] : y[(size_t)t * inner + i0 + i] * silu32(z);
        row_buf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float o = row_buf[i] * inv * to_float(w[i0 + i]);
        if (mode) o *= sigmoid32(to_float(src[(size_t)t * src_stride + z_col + i0 + i]));
        out[(size_t)t * inner + i0 + i] = from_float<TO>(o);
    }
}

// The same with a group's values in registers, eight a run (a group of a multiple of 8 features up to 8192, rows and
// the gate's columns on 16-byte boundaries): all loads of a thread are on their way together.
template <typename TI, typename TW, typename TO, int ITER>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_vec8_kernel(const float* __restrict__ y, const TI* __restrict__ src, int src_stride, int z_col,
                                const TW* __restrict__ w, float eps, TO* __restrict__ out, int inner, int groups, int mode) {
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y;
    const int gs = inner / groups, g8 = gs / 8;
    const int i0 = g * gs;
    float v[ITER][8], zg[ITER][8];
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int c = threadIdx.x + it * 256;
        if (c < g8) {
            load8(y + (size_t)t * inner + i0 + c * 8, v[it]);
            load8(src + (size_t)t * src_stride + z_col + i0 + c * 8, zg[it]);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (mode) zg[it][k] = sigmoid32(zg[it][k]); else { v[it][k] *= silu32(zg[it][k]); zg[it][k] = 1.0f; }
                ss += v[it][k] * v[it][k];
            }
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int c = threadIdx.x + it * 256;
        if (c < g8) {
            float wv[8], ov[8];
            load8(w + i0 + c * 8, wv);
#pragma unroll
            for (int k = 0; k < 8; ++k) ov[k] = v[it][k] * inv * wv[k] * zg[it][k];
            store8(out + (size_t)t * inner + i0 + c * 8, ov);
        }
    }
}

}  // namespace bg

using namespace bg;

extern "C" int bg_conv_silu(const void* src, int src_dtype, int src_stride, int col0, int channels, int taps, const void* w,
                            const void* b, int w_dtype, float* state, long long slot_stride, long long conv_off,
                            const int* slots, const int* row_req, const int* reqs, int n_req, float* out, int n_rows,
                            int act, const float* src_bias, cudaStream_t stream) {
    if (n_rows <= 0 || n_req <= 0) return BG_OK;
    if (channels <= 0 || taps < 1 || n_req > 65535) return BG_ERR_SHAPE;
    const unsigned bx = (unsigned)((channels + 127) / 128);
    if (bx > 65535) return BG_ERR_SHAPE;
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW,
        launch(conv_silu_kernel<TI, TW>, dim3(n_rows, bx), dim3(128), 0, stream, (const TI*)src, src_stride, col0, channels,
               taps, (const TW*)w, (const TW*)b, (const float*)state, (size_t)slot_stride, (size_t)conv_off, slots, row_req,
               reqs, out, act, src_bias)));
    BG_LAUNCH_CHECK();
    if (taps > 1) {
        BG_DISPATCH_DTYPE(src_dtype, TI,
            launch(conv_state_kernel<TI>, dim3(bx, n_req), dim3(128), 0, stream, (const TI*)src, src_stride, col0, channels,
                   taps, state, (size_t)slot_stride, (size_t)conv_off, slots, reqs, src_bias));
        BG_LAUNCH_CHECK();
    }
    return BG_OK;
}

// How the scan lays a head's state over CTAs: tiles of PT columns p, NS lanes per column (a power of two up to 32),
// each lane holding ceil(N / NS) values.  The tokens of a request come one after the other, so the time of a prompt
// is one CTA's time per token times the tokens.  What a token costs a thread besides its states (step size, input,
// the shuffles, the loop) is paid per thread, which speaks for many states a thread; the chain of dependent
// instructions of a token grows with them, which speaks for few: 8 states a thread set NS.  PT is the largest of
// 64, 32, 16, 8 that gives ONE request a CTA for every SM (heads x tiles).  The choice depends on the model's sizes
// alone, never on the step, so that a row's sums run in the same order in every step.
static int scan_layout(int H, int P, int N, int* pt_out, int* ns_out, int* npt_out) {
    if (P <= 0 || N <= 0) return BG_ERR_UNSUPPORTED;
    int ns = 1;
    while (ns < 32 && (N + ns - 1) / ns > 8) ns *= 2;
    const int npt = (N + ns - 1) / ns;
    if (npt > 64) return BG_ERR_UNSUPPORTED;
    const int sms = sm_count();
    int pt = 8;
    for (int cand = 64; cand >= 8; cand >>= 1)
        if (cand * ns <= SCAN_THREADS && (long long)H * ((P + cand - 1) / cand) >= sms) { pt = cand; break; }
    if (pt > P) pt = P;
    *pt_out = pt; *ns_out = ns; *npt_out = npt;
    return BG_OK;
}

extern "C" int bg_ssm_scan(const float* xbc, int channels, const void* src, int src_dtype, int src_stride, int dt_col,
                           const void* dt_bias, const void* A_log, const void* D, int w_dtype, float* state,
                           long long slot_stride, const int* slots, const int* reqs, int n_req, float* y, int H, int P,
                           int N, int G, cudaStream_t stream) {
    if (n_req <= 0) return BG_OK;
    if (H <= 0 || G <= 0 || H % G != 0 || n_req > 65535) return BG_ERR_SHAPE;
    int pt = 0, ns = 0, npt = 0;
    if (scan_layout(H, P, N, &pt, &ns, &npt) != BG_OK) return BG_ERR_UNSUPPORTED;
    const int threads = (pt * ns + 31) / 32 * 32;
    const int ptiles = (P + pt - 1) / pt;
    if (ptiles > 65535) return BG_ERR_UNSUPPORTED;
    const int npt_t = npt <= 1 ? 1 : npt <= 2 ? 2 : npt <= 4 ? 4 : npt <= 8 ? 8 : npt <= 16 ? 16 : npt <= 32 ? 32 : 64;
    const size_t smem = (size_t)(SCAN_CHUNK * (2 * (2 * npt_t * ns + pt + 2) + pt)) * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_UNSUPPORTED;
    dim3 grid(H, n_req, ptiles);
#define BG_SCAN(NPT)                                                                                                  \
    do {                                                                                                              \
        auto kern = ssm_scan_kernel<TI, TW, NPT>;                                                                     \
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch(kern, grid, dim3(threads), smem, stream, xbc, channels, (const TI*)src, src_stride, dt_col,            \
               (const TW*)dt_bias, (const TW*)A_log, (const TW*)D, state, (size_t)slot_stride, slots, reqs, y, H, P, N, G, ns, pt); \
    } while (0)
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW, {
        if (npt <= 1) BG_SCAN(1);
        else if (npt <= 2) BG_SCAN(2);
        else if (npt <= 4) BG_SCAN(4);
        else if (npt <= 8) BG_SCAN(8);
        else if (npt <= 16) BG_SCAN(16);
        else if (npt <= 32) BG_SCAN(32);
        else BG_SCAN(64);
    }));
#undef BG_SCAN
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_gated_group_rmsnorm(const float* y, const void* src, int src_dtype, int src_stride, int z_col, const void* w,
                                      int w_dtype, float eps, void* out, int out_dtype, int n_rows, int inner, int groups,
                                      int mode, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (groups <= 0 || inner % groups != 0 || groups > 65535) return BG_ERR_SHAPE;
    const int gs = inner / groups;
    const size_t smem = (size_t)gs * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    if (gs % 8 == 0 && gs <= 8192 && src_stride % 8 == 0 && z_col % 8 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)src % 16 == 0 &&
        (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const int iter = (gs / 8 + 255) / 256;
        BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(out_dtype, TO, {
            if (iter <= 1) launch(gated_group_rmsnorm_vec8_kernel<TI, TW, TO, 1>, dim3(n_rows, groups), dim3(256), 0, stream, y, (const TI*)src, src_stride, z_col, (const TW*)w, eps, (TO*)out, inner, groups, mode);
            else if (iter <= 2) launch(gated_group_rmsnorm_vec8_kernel<TI, TW, TO, 2>, dim3(n_rows, groups), dim3(256), 0, stream, y, (const TI*)src, src_stride, z_col, (const TW*)w, eps, (TO*)out, inner, groups, mode);
            else launch(gated_group_rmsnorm_vec8_kernel<TI, TW, TO, 4>, dim3(n_rows, groups), dim3(256), 0, stream, y, (const TI*)src, src_stride, z_col, (const TW*)w, eps, (TO*)out, inner, groups, mode);
        })));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    const int threads = gs >= 256 ? 256 : (gs + 31) / 32 * 32;
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(out_dtype, TO, {
        auto kern = gated_group_rmsnorm_kernel<TI, TW, TO>;
        if (smem > BG_SMEM_OPT_IN) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kern, dim3(n_rows, groups), dim3(threads), smem, stream, y, (const TI*)src, src_stride, z_col, (const TW*)w, eps,
               (TO*)out, inner, groups, mode);
    })));
    BG_LAUNCH_CHECK();
    return BG_OK;
}
