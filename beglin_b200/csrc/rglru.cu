// The real-gated linear recurrent unit: per channel c a state S_c that is carried from token to token,
//
//   r = sigmoid(gr + br),  i = sigmoid(gi + bi)        gr, gi: the gates' products of the convolved input u
//   log a = -C r softplus(lam_c),  a = e^(log a)
//   S <- a S + sqrt(1 - a^2) (i u),   out = S * gelu_tanh(y)      y: the other branch's product of the same token
//
// from S = 0 at a request's start (the first token is no special case).  Everything is float: the gates, the decay and
// its logarithm, the step and the state; 1 - a^2 is formed as -expm1(2 log a), which does not cancel for a near one.
//
//   rglru_scan          one thread per (request, channel) walks the request's rows of the step in order from the state
//                       in the request's slot and leaves the new state there.  Steps of single tokens and short portions.
//   rglru_scan_chunked  long portions: the rows of a request are cut into chunks; S_end = P S_begin + Q with
//                       P = prod a, Q the chunk's walk from zero, so (1) every (chunk, channel) forms P and Q, (2) a
//                       thread per channel walks the chunks of a request to every chunk's starting state, (3) every
//                       (chunk, channel) walks its rows again from that state and writes the outputs, with the rows' (a, b)
//                       as the first walk left them.  The two walks differ from the plain one by rounding only.
//
// The gates' products come as [blocks][T][2 bs]: for channel c = b bs + o the recurrence gate at [b][t][o] and the
// input gate at [b][t][bs + o].
#include "common.cuh"

namespace bg {

constexpr int LRU_THREADS = 128;

struct LruParams {
    const float* gates;     // [blocks][T][2 bs]
    const float* u;         // [T][W] the convolved input
    const float* src;       // the input product's rows; y of channel c at src[t * src_stride + y_col + c]
    int src_stride, y_col;
    const float* by;        // [W] or null: added to y before its activation
    const float* br;        // [W] bias of the recurrence gate
    const float* bi;        // [W] bias of the input gate
    const float* sp;        // [W] C * softplus(lam), made once when the model is built
    float* state;           // [slots][slot_stride], S in the first W values of a slot
    long long slot_stride;
    const int* slots;       // [requests]
    const int* reqs;        // [n][3] = (request, first row, rows)
    void* out;              // [T][W]
    int T, W, bs;
};

__device__ __forceinline__ float sigmoid32(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// (a, b) of S <- a S + b for row t of channel c.
__device__ __forceinline__ void lru_step(const LruParams& p, size_t gate_at, int t, int c, float brc, float bic, float spc, float* a,
                                         float* b) {
    const float r = sigmoid32(p.gates[gate_at] + brc);
    const float i = sigmoid32(p.gates[gate_at + p.bs] + bic);
    const float log_a = -r * spc;
    *a = expf(log_a);
    *b = sqrtf(-expm1f(2.0f * log_a)) * (i * p.u[(size_t)t * p.W + c]);
}

template <typename TO>
__global__ void __launch_bounds__(LRU_THREADS)
rglru_scan_kernel(LruParams p) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    if (c >= p.W) return;
    const int req = p.reqs[blockIdx.y * 3 + 0], row0 = p.reqs[blockIdx.y * 3 + 1], n = p.reqs[blockIdx.y * 3 + 2];
    if (n <= 0) return;
    const int blk = c / p.bs, o = c - blk * p.bs;
    const float brc = p.br[c], bic = p.bi[c], spc = p.sp[c];
    float* st = p.state + (size_t)p.slots[req] * p.slot_stride + c;
    float S = *st;
    TO* out = (TO*)p.out;
    const float yb = p.by ? p.by[c] : 0.0f;
    const size_t gbase = ((size_t)blk * p.T) * (2 * p.bs) + o;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        const int t = row0 + j;
        float a, b;
        lru_step(p, gbase + (size_t)t * (2 * p.bs), t, c, brc, bic, spc, &a, &b);
        S = fmaf(a, S, b);
        out[(size_t)t * p.W + c] = from_float<TO>(S * gelu_tanh32(p.src[(size_t)t * p.src_stride + p.y_col + c] + yb));
    }
    *st = S;
}

// chunks: [n][4] = (request, first row, rows, 0); longs: [n][4] = (request, first row, rows, index of its first chunk).
// pq: [chunks][2][W] = (P, Q) of a chunk; after the walk, [chunk][0] is the state at the chunk's start.
__global__ void __launch_bounds__(LRU_THREADS)
rglru_chunk_sums_kernel(LruParams p, const int* __restrict__ chunks, float* __restrict__ pq, float2* __restrict__ ab) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    if (c >= p.W) return;
    const int ch = blockIdx.y;
    const int row0 = chunks[ch * 4 + 1], n = chunks[ch * 4 + 2];
    const int blk = c / p.bs, o = c - blk * p.bs;
    const float brc = p.br[c], bic = p.bi[c], spc = p.sp[c];
    const size_t gbase = ((size_t)blk * p.T) * (2 * p.bs) + o;
    float P = 1.0f, Q = 0.0f;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        const int t = row0 + j;
        float a, b;
        lru_step(p, gbase + (size_t)t * (2 * p.bs), t, c, brc, bic, spc, &a, &b);
        ab[(size_t)t * p.W + c] = make_float2(a, b);
        P *= a;
        Q = fmaf(a, Q, b);
    }
    pq[((size_t)ch * 2 + 0) * p.W + c] = P;
    pq[((size_t)ch * 2 + 1) * p.W + c] = Q;
}

__global__ void __launch_bounds__(LRU_THREADS)
rglru_chunk_walk_kernel(LruParams p, const int* __restrict__ longs, int chunk_rows, float* __restrict__ pq) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    if (c >= p.W) return;
    const int req = longs[blockIdx.y * 4 + 0], n = longs[blockIdx.y * 4 + 2], first = longs[blockIdx.y * 4 + 3];
    const int n_chunks = (n + chunk_rows - 1) / chunk_rows;
    float* st = p.state + (size_t)p.slots[req] * p.slot_stride + c;
    float S = *st;
    // eight chunks' (P, Q) fetched at a time: the loads do not wait for the walk, only the eight products do
    for (int k0 = 0; k0 < n_chunks; k0 += 8) {
        float P[8], Q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const size_t at = ((size_t)(first + min(k0 + j, n_chunks - 1)) * 2) * p.W + c;
            P[j] = pq[at];
            Q[j] = pq[at + p.W];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (k0 + j < n_chunks) {
                pq[((size_t)(first + k0 + j) * 2) * p.W + c] = S;
                S = fmaf(P[j], S, Q[j]);
            }
        }
    }
    *st = S;
}

template <typename TO>
__global__ void __launch_bounds__(LRU_THREADS)
rglru_chunk_out_kernel(LruParams p, const int* __restrict__ chunks, const float* __restrict__ pq, const float2* __restrict__ ab) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * LRU_THREADS + threadIdx.x;
    if (c >= p.W) return;
    const int ch = blockIdx.y;
    const int row0 = chunks[ch * 4 + 1], n = chunks[ch * 4 + 2];
    TO* out = (TO*)p.out;
    const float yb = p.by ? p.by[c] : 0.0f;
    float S = pq[((size_t)ch * 2) * p.W + c];
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        const int t = row0 + j;
        const float2 s = ab[(size_t)t * p.W + c];              // (a, b) of the row, as the first walk formed them
        S = fmaf(s.x, S, s.y);
        out[(size_t)t * p.W + c] = from_float<TO>(S * gelu_tanh32(p.src[(size_t)t * p.src_stride + p.y_col + c] + yb));
    }
}

// u [T][W] float -> x2 [blocks][T][2 bs] bfloat16: per part the rounding of u to bfloat16 followed by the rounding of what
// the first rounding left out.  A product of x2 with a part's matrix repeated twice along its inner size is then the
// product of u itself to sixteen bits, with float accumulation, on the tensor cores.
__global__ void rglru_split_kernel(const float* __restrict__ u, __nv_bfloat16* __restrict__ x2, int T, int W, int bs) {
    pdl_launch();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * W) return;
    const int t = (int)(idx / W), c = (int)(idx - (size_t)t * W);
    const int blk = c / bs, o = c - blk * bs;
    const float v = u[idx];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
    __nv_bfloat16* dst = x2 + ((size_t)blk * T + t) * (2 * bs);
    dst[o] = hi;
    dst[bs + o] = lo;
}

// The same, four channels a thread (parts of a multiple of 4 channels): 16 bytes in, two stores of 8 bytes out.
__global__ void rglru_split_vec4_kernel(const float* __restrict__ u, __nv_bfloat16* __restrict__ x2, int T, int W, int bs) {
    pdl_launch();
    pdl_wait();
    const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (idx >= (size_t)T * W) return;
    const int t = (int)(idx / W), c = (int)(idx - (size_t)t * W);
    const int blk = c / bs, o = c - blk * bs;
    const float4 v = *reinterpret_cast<const float4*>(u + idx);
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
    __nv_bfloat16* dst = x2 + ((size_t)blk * T + t) * (2 * bs);
    uint2 hi, lo;
    hi.x = *reinterpret_cast<const unsigned*>(&h0); hi.y = *reinterpret_cast<const unsigned*>(&h1);
    lo.x = *reinterpret_cast<const unsigned*>(&l0); lo.y = *reinterpret_cast<const unsigned*>(&l1);
    *reinterpret_cast<uint2*>(dst + o) = hi;
    *reinterpret_cast<uint2*>(dst + bs + o) = lo;
}

// sp[c] = scale * softplus(lam[c]), float: log(1 + e^x), as x for large x.
template <typename TW>
__global__ void rglru_softplus_kernel(const TW* __restrict__ lam, float scale, float* __restrict__ sp, int W) {
    pdl_launch();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const float x = to_float(lam[c]);
    sp[c] = scale * (x > 20.0f ? x : log1pf(expf(x)));
}

}  // namespace bg

using namespace bg;

static int lru_params(LruParams* p, const float* gates, const float* u, const float* src, int src_stride, int y_col, const float* by,
                      const float* br,
                      const float* bi, const float* sp, float* state, long long slot_stride, const int* slots, void* out, int T,
                      int W, int blocks) {
    if (W <= 0 || blocks <= 0 || W % blocks != 0 || T <= 0) return BG_ERR_SHAPE;
    p->gates = gates; p->u = u; p->src = src; p->src_stride = src_stride; p->y_col = y_col; p->by = by; p->br = br; p->bi = bi; p->sp = sp;
    p->state = state; p->slot_stride = slot_stride; p->slots = slots; p->reqs = nullptr; p->out = out; p->T = T; p->W = W;
    p->bs = W / blocks;
    return BG_OK;
}

// The requests `reqs` [n_req][3] of a step walked row by row.
extern "C" int bg_rglru_scan(const float* gates, const float* u, const float* src, int src_stride, int y_col, const float* by,
                             const float* br,
                             const float* bi, const float* sp, float* state, long long slot_stride, const int* slots,
                             const int* reqs, int n_req, void* out, int out_dtype, int T, int W, int blocks, cudaStream_t stream) {
    if (n_req <= 0 || T <= 0) return BG_OK;
    if (n_req > 65535) return BG_ERR_SHAPE;
    LruParams p;
    const int rc = lru_params(&p, gates, u, src, src_stride, y_col, by, br, bi, sp, state, slot_stride, slots, out, T, W, blocks);
    if (rc != BG_OK) return rc;
    p.reqs = reqs;
    const dim3 grid((W + LRU_THREADS - 1) / LRU_THREADS, n_req);
    BG_DISPATCH_DTYPE(out_dtype, TO, launch(rglru_scan_kernel<TO>, grid, dim3(LRU_THREADS), 0, stream, p));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// The long requests of a step in chunks of `chunk_rows` rows: chunks [n_chunks][4], longs [n_long][4], pq float
// [n_chunks][2][W] and ab float [T][W][2] of the caller's.
extern "C" int bg_rglru_scan_chunked(const float* gates, const float* u, const float* src, int src_stride, int y_col,
                                     const float* by, const float* br, const float* bi, const float* sp, float* state, long long slot_stride,
                                     const int* slots, const int* chunks, int n_chunks, const int* longs, int n_long,
                                     int chunk_rows, float* pq, float* ab, void* out, int out_dtype, int T, int W, int blocks,
                                     cudaStream_t stream) {
    if (n_chunks <= 0 || n_long <= 0 || T <= 0) return BG_OK;
    if (n_chunks > 65535 || n_long > 65535 || chunk_rows <= 0) return BG_ERR_SHAPE;
    LruParams p;
    const int rc = lru_params(&p, gates, u, src, src_stride, y_col, by, br, bi, sp, state, slot_stride, slots, out, T, W, blocks);
    if (rc != BG_OK) return rc;
    const unsigned bx = (W + LRU_THREADS - 1) / LRU_THREADS;
    launch(rglru_chunk_sums_kernel, dim3(bx, n_chunks), dim3(LRU_THREADS), 0, stream, p, chunks, pq, (float2*)ab);
    BG_LAUNCH_CHECK();
    launch(rglru_chunk_walk_kernel, dim3(bx, n_long), dim3(LRU_THREADS), 0, stream, p, longs, chunk_rows, pq);
    BG_LAUNCH_CHECK();
    BG_DISPATCH_DTYPE(out_dtype, TO, launch(rglru_chunk_out_kernel<TO>, dim3(bx, n_chunks), dim3(LRU_THREADS), 0, stream, p, chunks,
                                            (const float*)pq, (const float2*)ab));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_rglru_split(const float* u, void* x2, int T, int W, int blocks, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (W <= 0 || blocks <= 0 || W % blocks != 0) return BG_ERR_SHAPE;
    const size_t n = (size_t)T * W;
    if ((W / blocks) % 4 == 0 && (uintptr_t)u % 16 == 0 && (uintptr_t)x2 % 8 == 0) {
        launch(rglru_split_vec4_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, u, (__nv_bfloat16*)x2, T, W,
               W / blocks);
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    launch(rglru_split_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, u, (__nv_bfloat16*)x2, T, W, W / blocks);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_rglru_softplus(const void* lam, int lam_dtype, float scale, float* sp, int W, cudaStream_t stream) {
    if (W <= 0) return BG_OK;
    BG_DISPATCH_DTYPE(lam_dtype, TW, launch(rglru_softplus_kernel<TW>, dim3((W + 255) / 256), dim3(256), 0, stream, (const TW*)lam,
                                            scale, sp, W));
    BG_LAUNCH_CHECK();
    return BG_OK;
}
