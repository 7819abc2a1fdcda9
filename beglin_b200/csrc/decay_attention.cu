// Linear attention with a constant decay per head, and the sum that joins the branches of a layer.
//
// Per head, with q, k (n features) and v (nv features) of a token, all three silu of a product of the mixer's input:
//     S <- d S + k v^T        (S is n x nv, float, one per request and head, zero when the request starts)
//     o  = S^T q
// The state is carried from step to step in a slot of the cache manager's slab.  Everything is float: the state, the
// decay, the products that enter it and the readout.  Three kernels:
//   decay_attention_reg_kernel    blocks per (head, request, 32 columns of the state) walk the request's tokens in turn,
//                                 the state in registers.  For steps of single tokens and short portions.
//   decay_attention_seq_kernel    the same walk with a head's whole state in shared memory, one block per (head,
//                                 request): for heads of more rows than the registers take.
//   decay_attention_chunk_*       long portions, cut into chunks of DC tokens: the chunks' own sums of decayed k v^T in
//                                 parallel, a short pass over the chunks that turns them into the states at the chunks'
//                                 starts, then every chunk's outputs in parallel (the earlier chunks through the state,
//                                 the chunk's own tokens through their decayed scores).
#include "common.cuh"

namespace bg {

__device__ __forceinline__ float da_silu(float z) { return z / (1.0f + expf(-z)); }

struct DecayAttnParams {
    const void* src; int src_stride; int parts; size_t part_stride;   // rows [.. q .. k .. v ..] or their partial sums
    int q_col, k_col, v_col;
    const float* decay;                                               // [H]
    float* state; size_t slot_stride;                                 // slab [slots][>= H * n * nv]
    const int* slots;                                                 // [requests]
    const int* reqs;                                                  // [n_req][3] = (request, first row, rows)
    float* y;                                                         // [T][H * nv]
    int H, n, nv;
};

template <typename TS>
__global__ void __launch_bounds__(256) decay_attention_seq_kernel(DecayAttnParams p) {
    extern __shared__ float da_s[];
    const int n = p.n, nv = p.nv;
    float* S = da_s;                       // [n][nv]
    float* qs = S + (size_t)n * nv;        // [n]
    float* ks = qs + n;                    // [n]
    float* vs = ks + n;                    // [nv]
    float* red = vs + nv;                  // [slices][nv]
    pdl_launch();
    const int h = blockIdx.x, r = blockIdx.y;
    const int req = p.reqs[r * 3 + 0], row0 = p.reqs[r * 3 + 1], rows = p.reqs[r * 3 + 2];
    const int tid = threadIdx.x;
    const int slices = nv <= (int)blockDim.x ? (int)blockDim.x / nv : 1;
    const float d = p.decay[h];
    pdl_wait();
    if (rows <= 0) return;
    float* st = p.state + (size_t)p.slots[req] * p.slot_stride + (size_t)h * n * nv;
    for (int i = tid; i < n * nv; i += blockDim.x) S[i] = st[i];
    const TS* src = (const TS*)p.src;
    for (int t = 0; t < rows; ++t) {
        const TS* row = src + (size_t)(row0 + t) * p.src_stride;
        __syncthreads();
        for (int i = tid; i < n; i += blockDim.x) {
            qs[i] = da_silu(sum_parts(row + p.q_col + h * n + i, p.parts, p.part_stride));
            ks[i] = da_silu(sum_parts(row + p.k_col + h * n + i, p.parts, p.part_stride));
        }
        for (int i = tid; i < nv; i += blockDim.x) vs[i] = da_silu(sum_parts(row + p.v_col + h * nv + i, p.parts, p.part_stride));
        __syncthreads();
        for (int c0 = 0; c0 < nv; c0 += blockDim.x) {           // (one pass unless values are wider than the block)
            const int sl = nv <= (int)blockDim.x ? tid / nv : 0;
            const int c = nv <= (int)blockDim.x ? tid - sl * nv : c0 + tid;
            if (c < nv && sl < slices) {
                const float v = vs[c];
                float acc = 0.0f;
                for (int i = sl; i < n; i += slices) {
                    const float s = fmaf(d, S[(size_t)i * nv + c], ks[i] * v);
                    S[(size_t)i * nv + c] = s;
                    acc = fmaf(s, qs[i], acc);
                }
                red[(size_t)sl * nv + c] = acc;
            }
        }
        __syncthreads();
        for (int c = tid; c < nv; c += blockDim.x) {
            float acc = 0.0f;
            for (int sl = 0; sl < slices; ++sl) acc += red[(size_t)sl * nv + c];
            p.y[(size_t)(row0 + t) * p.H * nv + (size_t)h * nv + c] = acc;
        }
    }
    __syncthreads();
    for (int i = tid; i < n * nv; i += blockDim.x) st[i] = S[i];
}

// The same walk with the state in registers: a block takes DA_COLS columns of one head's state (of one request), thread
// (slice, column) holds the rows slice, slice + slices, ... of its column, at most R of them.  A head of nv columns is
// spread over nv / DA_COLS blocks, which share nothing: a column's sum over the rows stays inside its block.
constexpr int DA_COLS = 32;

template <typename TS, int R>
__global__ void __launch_bounds__(256) decay_attention_reg_kernel(DecayAttnParams p) {
    extern __shared__ float da_s[];
    const int n = p.n, nv = p.nv;
    const int cols = nv < DA_COLS ? nv : DA_COLS;
    const int slices = (int)blockDim.x / cols;
    float* qs = da_s;                      // [n]
    float* ks = qs + n;                    // [n]
    float* vs = ks + n;                    // [cols]
    float* red = vs + cols;                // [slices][cols]
    pdl_launch();
    const int h = blockIdx.x, r = blockIdx.y, col0 = blockIdx.z * cols;
    const int req = p.reqs[r * 3 + 0], row0 = p.reqs[r * 3 + 1], rows = p.reqs[r * 3 + 2];
    const int tid = threadIdx.x;
    const int sl = tid / cols, c = tid - sl * cols;
    const bool own = sl < slices && col0 + c < nv;
    const float d = p.decay[h];
    pdl_wait();
    if (rows <= 0) return;
    float* st = p.state + (size_t)p.slots[req] * p.slot_stride + (size_t)h * n * nv + col0 + c;
    float S[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int i = sl + k * slices;
        S[k] = (own && i < n) ? st[(size_t)i * nv] : 0.0f;
    }
    const TS* src = (const TS*)p.src;
    for (int t = 0; t < rows; ++t) {
        const TS* row = src + (size_t)(row0 + t) * p.src_stride;
        __syncthreads();
        for (int i = tid; i < n; i += blockDim.x) {
            qs[i] = da_silu(sum_parts(row + p.q_col + h * n + i, p.parts, p.part_stride));
            ks[i] = da_silu(sum_parts(row + p.k_col + h * n + i, p.parts, p.part_stride));
        }
        if (tid < cols && col0 + tid < nv) vs[tid] = da_silu(sum_parts(row + p.v_col + h * nv + col0 + tid, p.parts, p.part_stride));
        __syncthreads();
        if (own) {
            const float v = vs[c];
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const int i = sl + k * slices;
                if (i < n) {
                    S[k] = fmaf(d, S[k], ks[i] * v);
                    acc = fmaf(S[k], qs[i], acc);
                }
            }
            red[sl * cols + c] = acc;
        }
        __syncthreads();
        if (tid < cols && col0 + tid < nv) {
            float acc = 0.0f;
            for (int q = 0; q < slices; ++q) acc += red[q * cols + tid];
            p.y[(size_t)(row0 + t) * p.H * nv + (size_t)h * nv + col0 + tid] = acc;
        }
    }
    if (own) {
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int i = sl + k * slices;
            if (i < n) st[(size_t)i * nv] = S[k];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Long portions in chunks of DC tokens.  With S the state at a chunk's start, r its number of tokens and t, j = 0 .. r-1:
//     o_t     = d^(t+1) S^T q_t + sum_{j <= t} d^(t-j) (q_t . k_j) v_j
//     S_next  = d^r S + A,    A = sum_j d^(r-1-j) k_j v_j^T
// decay_chunk_sum_kernel    A of every chunk (a block per head and chunk)
// decay_chunk_scan_kernel   a thread per element of the state walks its request's chunks: A is replaced by the state at
//                           the chunk's start, the request's slot gets the state behind its last chunk
// decay_chunk_out_kernel    o of every chunk (a block per head and chunk): scores of the chunk's own tokens times their
//                           powers of d, then both sums
// Powers of d come from one table made by repeated multiplication, so d = 0 and d = 1 need no logarithm.  Threads own
// 4 x 4 tiles of outputs; rows of shared memory are padded to multiples of four floats and read as float4.
constexpr int DC = 64;                    // tokens of a chunk
constexpr int DCP = DC + 4;               // row stride of the transposed tiles [feature][token]

struct DecayChunkParams {
    const void* src; int src_stride; int parts; size_t part_stride;
    int q_col, k_col, v_col;
    const float* decay;
    float* state; size_t slot_stride; const int* slots;
    const int* chunks;                    // [n_chunks][4] = (request, first row, rows, -)
    const int* longs;                     // [n_long][4]   = (request, first row, rows, first chunk)
    float* work;                          // [n_chunks][H][n * nv]
    float* y;
    int H, n, nv, np, nvp;                // np, nvp: n, nv rounded up to multiples of 4
};

__device__ __forceinline__ void decay_powers(float* pw, float d) {      // pw[k] = d^k, k = 0 .. DC
    if (threadIdx.x == 0) {
        float v = 1.0f;
        for (int k = 0; k <= DC; ++k) { pw[k] = v; v *= d; }
    }
}

#define DA_FMA44(acc, a, b)                                                                                      \
    do {                                                                                                         \
        acc[0][0] = fmaf(a.x, b.x, acc[0][0]); acc[0][1] = fmaf(a.x, b.y, acc[0][1]); acc[0][2] = fmaf(a.x, b.z, acc[0][2]); acc[0][3] = fmaf(a.x, b.w, acc[0][3]); \
        acc[1][0] = fmaf(a.y, b.x, acc[1][0]); acc[1][1] = fmaf(a.y, b.y, acc[1][1]); acc[1][2] = fmaf(a.y, b.z, acc[1][2]); acc[1][3] = fmaf(a.y, b.w, acc[1][3]); \
        acc[2][0] = fmaf(a.z, b.x, acc[2][0]); acc[2][1] = fmaf(a.z, b.y, acc[2][1]); acc[2][2] = fmaf(a.z, b.z, acc[2][2]); acc[2][3] = fmaf(a.z, b.w, acc[2][3]); \
        acc[3][0] = fmaf(a.w, b.x, acc[3][0]); acc[3][1] = fmaf(a.w, b.y, acc[3][1]); acc[3][2] = fmaf(a.w, b.z, acc[3][2]); acc[3][3] = fmaf(a.w, b.w, acc[3][3]); \
    } while (0)


// Fills of shared memory from the rows of a chunk go eight loads at a time per thread: the loads of a batch are in
// flight together, and the activations follow when they have landed.
constexpr int DA_BATCH = 8;
constexpr int DC_THREADS = 512;

// The (row, column) of element tid + k * blockDim.x of a [rows][w] tile, stepped without a division per element.
struct TileWalk {
    int j, i, dj, di, w;
    __device__ __forceinline__ TileWalk(int w_) : w(w_) {
        j = (int)threadIdx.x / w; i = (int)threadIdx.x - j * w;
        dj = (int)blockDim.x / w; di = (int)blockDim.x - dj * w;
    }
    __device__ __forceinline__ void next() { i += di; j += dj; if (i >= w) { i -= w; ++j; } }
};

template <typename TS>
__global__ void __launch_bounds__(DC_THREADS) decay_chunk_sum_kernel(DecayChunkParams p) {
    extern __shared__ __align__(16) float dc_s[];
    const int n = p.n, nv = p.nv, np = p.np, nvp = p.nvp;
    float* Ks = dc_s;                          // [DC][np], k_j times d^(r-1-j)
    float* Vs = Ks + (size_t)DC * np;          // [DC][nvp]
    float* pw = Vs + (size_t)DC * nvp;         // [DC + 1]
    pdl_launch();
    const int h = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
    decay_powers(pw, p.decay[h]);
    pdl_wait();
    const int row0 = p.chunks[c * 4 + 1], rows = p.chunks[c * 4 + 2];
    __syncthreads();
    const TS* src = (const TS*)p.src;
    for (TileWalk w(np); w.j < DC;) {
        float raw[DA_BATCH];
        int jj[DA_BATCH], ii[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            jj[u] = w.j; ii[u] = w.i; w.next();
            raw[u] = (jj[u] < rows && ii[u] < n) ? sum_parts(src + (size_t)(row0 + jj[u]) * p.src_stride + p.k_col + h * n + ii[u], p.parts, p.part_stride) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (jj[u] < DC) Ks[jj[u] * np + ii[u]] = raw[u] == -INFINITY ? 0.0f : da_silu(raw[u]) * pw[rows - 1 - jj[u]];
    }
    for (TileWalk w(nvp); w.j < DC;) {
        float raw[DA_BATCH];
        int jj[DA_BATCH], ii[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            jj[u] = w.j; ii[u] = w.i; w.next();
            raw[u] = (jj[u] < rows && ii[u] < nv) ? sum_parts(src + (size_t)(row0 + jj[u]) * p.src_stride + p.v_col + h * nv + ii[u], p.parts, p.part_stride) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (jj[u] < DC) Vs[jj[u] * nvp + ii[u]] = raw[u] == -INFINITY ? 0.0f : da_silu(raw[u]);
    }
    __syncthreads();
    float* A = p.work + ((size_t)c * p.H + h) * n * nv;
    const int tc = nvp / 4, tiles = (np / 4) * tc;
    for (int tile = tid; tile < tiles; tile += blockDim.x) {
        const int i0 = (tile / tc) * 4, c0 = (tile % tc) * 4;
        float acc[4][4] = {};
        for (int j = 0; j < rows; ++j) {
            const float4 kk = *(const float4*)(Ks + (size_t)j * np + i0);
            const float4 vv = *(const float4*)(Vs + (size_t)j * nvp + c0);
            DA_FMA44(acc, kk, vv);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (i0 + a < n && c0 + b < nv) A[(size_t)(i0 + a) * nv + c0 + b] = acc[a][b];
    }
}

__global__ void __launch_bounds__(256) decay_chunk_scan_kernel(DecayChunkParams p) {
    pdl_launch();
    pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, l = blockIdx.z;
    const int sz = p.n * p.nv;
    if (e >= sz) return;
    const int req = p.longs[l * 4 + 0], rows = p.longs[l * 4 + 2], c0 = p.longs[l * 4 + 3];
    const int n_chunks = (rows + DC - 1) / DC, last_rows = rows - (n_chunks - 1) * DC;
    const float d = p.decay[h];
    float dfull = 1.0f, dlast = 1.0f;
    for (int k = 0; k < DC; ++k) { dfull *= d; if (k + 1 == last_rows) dlast = dfull; }
    float* st = p.state + (size_t)p.slots[req] * p.slot_stride + (size_t)h * sz + e;
    float* a0 = p.work + ((size_t)c0 * p.H + h) * sz + e;
    const size_t step = (size_t)p.H * sz;
    float S = *st;
    // the chunks' sums are fetched eight at a time, so that the walk waits for memory once per batch and not per chunk
    for (int c = 0; c < n_chunks; c += DA_BATCH) {
        float A[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) A[u] = c + u < n_chunks ? a0[(size_t)(c + u) * step] : 0.0f;
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (c + u < n_chunks) {
                a0[(size_t)(c + u) * step] = S;
                S = fmaf(c + u == n_chunks - 1 ? dlast : dfull, S, A[u]);
            }
    }
    *st = S;
}

template <typename TS>
__global__ void __launch_bounds__(DC_THREADS) decay_chunk_out_kernel(DecayChunkParams p) {
    extern __shared__ __align__(16) float dc_s[];
    const int n = p.n, nv = p.nv, np = p.np, nvp = p.nvp;
    float* Qt = dc_s;                          // [np][DCP]
    float* Kt = Qt + (size_t)np * DCP;         // [np][DCP]
    float* Vs = Kt + (size_t)np * DCP;         // [DC][nvp]
    float* Ss = Vs + (size_t)DC * nvp;         // [np][nvp]
    float* Pt = Ss + (size_t)np * nvp;         // [DC (key)][DCP (query)]
    float* pw = Pt + (size_t)DC * DCP;         // [DC + 1]
    pdl_launch();
    const int h = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
    decay_powers(pw, p.decay[h]);
    pdl_wait();
    const int row0 = p.chunks[c * 4 + 1], rows = p.chunks[c * 4 + 2];
    const TS* src = (const TS*)p.src;
    for (TileWalk w(np); w.j < DC;) {
        float rq[DA_BATCH], rk[DA_BATCH];
        int jj[DA_BATCH], ii[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            jj[u] = w.j; ii[u] = w.i; w.next();
            rq[u] = rk[u] = -INFINITY;
            if (jj[u] < rows && ii[u] < n) {
                const TS* row = src + (size_t)(row0 + jj[u]) * p.src_stride + h * n + ii[u];
                rq[u] = sum_parts(row + p.q_col, p.parts, p.part_stride);
                rk[u] = sum_parts(row + p.k_col, p.parts, p.part_stride);
            }
        }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (jj[u] < DC) {
                Qt[(size_t)ii[u] * DCP + jj[u]] = rq[u] == -INFINITY ? 0.0f : da_silu(rq[u]);
                Kt[(size_t)ii[u] * DCP + jj[u]] = rk[u] == -INFINITY ? 0.0f : da_silu(rk[u]);
            }
    }
    for (TileWalk w(nvp); w.j < DC;) {
        float raw[DA_BATCH];
        int jj[DA_BATCH], ii[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            jj[u] = w.j; ii[u] = w.i; w.next();
            raw[u] = (jj[u] < rows && ii[u] < nv) ? sum_parts(src + (size_t)(row0 + jj[u]) * p.src_stride + p.v_col + h * nv + ii[u], p.parts, p.part_stride) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (jj[u] < DC) Vs[jj[u] * nvp + ii[u]] = raw[u] == -INFINITY ? 0.0f : da_silu(raw[u]);
    }
    const float* S0 = p.work + ((size_t)c * p.H + h) * n * nv;
    for (TileWalk w(nvp); w.j < np;) {
        float raw[DA_BATCH];
        int jj[DA_BATCH], ii[DA_BATCH];
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u) {
            jj[u] = w.j; ii[u] = w.i; w.next();
            raw[u] = (jj[u] < n && ii[u] < nv) ? S0[(size_t)jj[u] * nv + ii[u]] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < DA_BATCH; ++u)
            if (jj[u] < np) Ss[jj[u] * nvp + ii[u]] = raw[u];
    }
    __syncthreads();
    // scores of the chunk's own tokens: a 4 x 4 tile (queries t0.., keys j0..) per thread
    for (int tile = tid; tile < (DC / 4) * (DC / 4); tile += blockDim.x) {
        const int t0 = (tile / (DC / 4)) * 4, j0 = (tile % (DC / 4)) * 4;
        float acc[4][4] = {};
        if (j0 <= t0 + 3 && j0 < rows && t0 < rows) {
            for (int i = 0; i < n; ++i) {
                const float4 qq = *(const float4*)(Qt + (size_t)i * DCP + t0);
                const float4 kk = *(const float4*)(Kt + (size_t)i * DCP + j0);
                DA_FMA44(acc, qq, kk);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int t = t0 + a, j = j0 + b;
                Pt[(size_t)j * DCP + t] = j <= t ? acc[a][b] * pw[t - j] : 0.0f;
            }
    }
    __syncthreads();
    const int tc = nvp / 4, tiles = (DC / 4) * tc;
    for (int tile = tid; tile < tiles; tile += blockDim.x) {
        const int t0 = (tile / tc) * 4, c0 = (tile % tc) * 4;
        if (t0 >= rows) continue;
        float acc[4][4] = {};
        for (int i = 0; i < n; ++i) {
            const float4 qq = *(const float4*)(Qt + (size_t)i * DCP + t0);
            const float4 ss = *(const float4*)(Ss + (size_t)i * nvp + c0);
            DA_FMA44(acc, qq, ss);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float w = pw[t0 + a + 1];
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] *= w;
        }
        const int jend = min(rows, t0 + 4);
        for (int j = 0; j < jend; ++j) {
            const float4 pp = *(const float4*)(Pt + (size_t)j * DCP + t0);
            const float4 vv = *(const float4*)(Vs + (size_t)j * nvp + c0);
            DA_FMA44(acc, pp, vv);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (t0 + a < rows && c0 + b < nv)
                    p.y[(size_t)(row0 + t0 + a) * p.H * nv + (size_t)h * nv + c0 + b] = acc[a][b];
    }
}

static size_t decay_chunk_out_smem(int np, int nvp) {
    return ((size_t)2 * np * DCP + (size_t)DC * nvp + (size_t)np * nvp + (size_t)DC * DCP + DC + 4) * sizeof(float);
}

// ---------------------------------------------------------------------------------------------------------------
// x[t] (= or +=) sum_i scale_i * term_i[t], term_i a [T, d] tensor of either type or the float partial sums of a
// split product; then, when asked, the rows of x RMS-normed with one or two weight vectors (the two norms of a layer
// whose sublayers read the same stream share the statistics).  The sum and the statistics are float.
constexpr int MAX_TERMS = 6;
struct TermsParams {
    float* x;
    const void* term[MAX_TERMS]; int dtype[MAX_TERMS]; int parts[MAX_TERMS]; size_t part_stride[MAX_TERMS]; float scale[MAX_TERMS];
    int n_terms, assign;
    const void* w1; const void* w2; int w_dtype; float eps;
    void* out1; void* out2; int out_dtype;
    int d;
};

__device__ __forceinline__ float term_value(const TermsParams& p, int i, size_t at) {
    if (p.dtype[i] == BG_DTYPE_F32) return sum_parts((const float*)p.term[i] + at, p.parts[i], p.part_stride[i]);
    return sum_parts((const __nv_bfloat16*)p.term[i] + at, p.parts[i], p.part_stride[i]);
}
__device__ __forceinline__ float weight_value(const void* w, int dtype, int i) {
    return dtype == BG_DTYPE_F32 ? ((const float*)w)[i] : __bfloat162float(((const __nv_bfloat16*)w)[i]);
}
__device__ __forceinline__ void store_value(void* out, int dtype, size_t at, float v) {
    if (dtype == BG_DTYPE_F32) ((float*)out)[at] = v; else ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(v);
}

__global__ void __launch_bounds__(256) add_terms_norm_kernel(TermsParams p) {
    extern __shared__ float row_s[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const size_t t = blockIdx.x;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < p.d; j += blockDim.x) {
        const size_t at = t * p.d + j;
        float v = p.assign ? 0.0f : p.x[at];
        for (int i = 0; i < p.n_terms; ++i) v = fmaf(p.scale[i], term_value(p, i, at), v);
        if (p.n_terms > 0 || p.assign) p.x[at] = v;
        row_s[j] = v;
        ss += v * v;
    }
    if (!p.out1) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)p.d + p.eps);
    for (int j = threadIdx.x; j < p.d; j += blockDim.x) {
        const float v = row_s[j] * inv;
        store_value(p.out1, p.out_dtype, t * p.d + j, v * weight_value(p.w1, p.w_dtype, j));
        if (p.out2) store_value(p.out2, p.out_dtype, t * p.d + j, v * weight_value(p.w2, p.w_dtype, j));
    }
}

// The same, four columns a thread at a time (d a multiple of 4, every pointer 16-byte aligned): the terms are walked
// outside the columns, so a term's type and its number of partial sums are looked at once per group of four.
__global__ void __launch_bounds__(1024) add_terms_norm_vec4_kernel(TermsParams p) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int d4 = p.d >> 2;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < d4; j += blockDim.x) {
        const size_t at = t * p.d + (size_t)j * 4;
        float4 v = p.assign ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : *reinterpret_cast<const float4*>(p.x + at);
        for (int i = 0; i < p.n_terms; ++i) {
            const float sc = p.scale[i];
            if (p.dtype[i] == BG_DTYPE_F32) {
                const float* base = (const float*)p.term[i] + at;
#pragma unroll 4
                for (int q = 0; q < p.parts[i]; ++q) {
                    const float4 a = *reinterpret_cast<const float4*>(base + (size_t)q * p.part_stride[i]);
                    v.x = fmaf(sc, a.x, v.x); v.y = fmaf(sc, a.y, v.y); v.z = fmaf(sc, a.z, v.z); v.w = fmaf(sc, a.w, v.w);
                }
            } else {
                const __nv_bfloat16* base = (const __nv_bfloat16*)p.term[i] + at;
#pragma unroll 4
                for (int q = 0; q < p.parts[i]; ++q) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(base + (size_t)q * p.part_stride[i]);
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v.x = fmaf(sc, lo.x, v.x); v.y = fmaf(sc, lo.y, v.y); v.z = fmaf(sc, hi.x, v.z); v.w = fmaf(sc, hi.y, v.w);
                }
            }
        }
        if (p.n_terms > 0 || p.assign) *reinterpret_cast<float4*>(p.x + at) = v;
        *reinterpret_cast<float4*>(row_s + (size_t)j * 4) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (!p.out1) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)p.d + p.eps);
    for (int j = threadIdx.x; j < d4; j += blockDim.x) {
        const float4 v = *reinterpret_cast<const float4*>(row_s + (size_t)j * 4);
        const float r[4] = {v.x * inv, v.y * inv, v.z * inv, v.w * inv};
        const size_t at = t * p.d + (size_t)j * 4;
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            void* out = o == 0 ? p.out1 : p.out2;
            const void* w = o == 0 ? p.w1 : p.w2;
            if (!out) continue;
            float y[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) y[k] = r[k] * weight_value(w, p.w_dtype, j * 4 + k);
            if (p.out_dtype == BG_DTYPE_F32) {
                *reinterpret_cast<float4*>((float*)out + at) = make_float4(y[0], y[1], y[2], y[3]);
            } else {
                __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
                uint2 pack;
                pack.x = *reinterpret_cast<unsigned*>(&a); pack.y = *reinterpret_cast<unsigned*>(&b);
                *reinterpret_cast<uint2*>((__nv_bfloat16*)out + at) = pack;
            }
        }
    }
}

}  // namespace bg

using namespace bg;

extern "C" int bg_decay_attention(const void* src, int src_dtype, int src_stride, int parts, long long part_stride, int q_col,
                                  int k_col, int v_col, const float* decay, float* state, long long slot_stride, const int* slots,
                                  const int* reqs, int n_req, float* y, int H, int n, int nv, cudaStream_t stream) {
    if (n_req <= 0) return BG_OK;
    if (H <= 0 || n <= 0 || nv <= 0 || parts < 1 || n_req > 65535) return BG_ERR_SHAPE;
    DecayAttnParams p;
    p.src = src; p.src_stride = src_stride; p.parts = parts; p.part_stride = (size_t)part_stride; p.q_col = q_col; p.k_col = k_col;
    p.v_col = v_col; p.decay = decay; p.state = state; p.slot_stride = (size_t)slot_stride; p.slots = slots; p.reqs = reqs; p.y = y;
    p.H = H; p.n = n; p.nv = nv;
    const int threads = 256;
    // the state in registers where a thread's share of a column fits (heads of up to 256 rows), else in shared memory
    const int cols = nv < DA_COLS ? nv : DA_COLS, rslices = threads / cols, per_thread = (n + rslices - 1) / rslices;
    if (per_thread <= 32 && (nv + cols - 1) / cols <= 65535) {
        const size_t rsmem = ((size_t)2 * n + cols + (size_t)rslices * cols) * sizeof(float);
        const dim3 grid(H, n_req, (nv + cols - 1) / cols);
        BG_DISPATCH_DTYPE(src_dtype, TS, {
            if (per_thread <= 16) launch(decay_attention_reg_kernel<TS, 16>, grid, dim3(threads), rsmem, stream, p);
            else launch(decay_attention_reg_kernel<TS, 32>, grid, dim3(threads), rsmem, stream, p);
        });
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    const int slices = nv <= threads ? threads / nv : 1;
    const size_t smem = ((size_t)n * nv + 2 * n + nv + (size_t)slices * nv) * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_UNSUPPORTED;
    BG_DISPATCH_DTYPE(src_dtype, TS, {
        auto kern = decay_attention_seq_kernel<TS>;
        if (smem > BG_SMEM_OPT_IN) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        launch(kern, dim3(H, n_req), dim3(threads), smem, stream, p);
    });
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// 0 when the chunked kernels take heads of n x nv values (their tiles fit in shared memory), else BG_ERR_UNSUPPORTED.
extern "C" int bg_decay_attention_chunk_plan(int n, int nv, int* chunk) {
    if (n <= 0 || nv <= 0) return BG_ERR_SHAPE;
    const int np = (n + 3) / 4 * 4, nvp = (nv + 3) / 4 * 4;
    if (chunk) *chunk = DC;
    return decay_chunk_out_smem(np, nvp) <= 200 * 1024 ? BG_OK : BG_ERR_UNSUPPORTED;
}

// The chunked form for requests of many rows.  chunks [n_chunks][4] = (request, first row, rows <= chunk, -) lists every
// long request's chunks in turn; longs [n_long][4] = (request, first row, rows, index of its first chunk); work is
// float [n_chunks][H][n * nv].
extern "C" int bg_decay_attention_chunked(const void* src, int src_dtype, int src_stride, int parts, long long part_stride,
                                          int q_col, int k_col, int v_col, const float* decay, float* state, long long slot_stride,
                                          const int* slots, const int* chunks, int n_chunks, const int* longs, int n_long,
                                          float* work, float* y, int H, int n, int nv, cudaStream_t stream) {
    if (n_chunks <= 0 || n_long <= 0) return BG_OK;
    if (H <= 0 || n <= 0 || nv <= 0 || parts < 1 || n_chunks > 65535 || n_long > 65535 || H > 65535) return BG_ERR_SHAPE;
    DecayChunkParams p;
    p.src = src; p.src_stride = src_stride; p.parts = parts; p.part_stride = (size_t)part_stride; p.q_col = q_col; p.k_col = k_col;
    p.v_col = v_col; p.decay = decay; p.state = state; p.slot_stride = (size_t)slot_stride; p.slots = slots; p.chunks = chunks;
    p.longs = longs; p.work = work; p.y = y; p.H = H; p.n = n; p.nv = nv; p.np = (n + 3) / 4 * 4; p.nvp = (nv + 3) / 4 * 4;
    const size_t smem_sum = ((size_t)DC * p.np + (size_t)DC * p.nvp + DC + 4) * sizeof(float);
    const size_t smem_out = decay_chunk_out_smem(p.np, p.nvp);
    if (smem_out > 200 * 1024 || smem_sum > 200 * 1024) return BG_ERR_UNSUPPORTED;
    BG_DISPATCH_DTYPE(src_dtype, TS, {
        auto ksum = decay_chunk_sum_kernel<TS>;
        auto kout = decay_chunk_out_kernel<TS>;
        if (smem_sum > BG_SMEM_OPT_IN) {
            cudaError_t e = cudaFuncSetAttribute(ksum, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_sum);
            if (e != cudaSuccess) return (int)e;
        }
        if (smem_out > BG_SMEM_OPT_IN) {
            cudaError_t e = cudaFuncSetAttribute(kout, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
            if (e != cudaSuccess) return (int)e;
        }
        launch(ksum, dim3(H, n_chunks), dim3(DC_THREADS), smem_sum, stream, p);
        BG_LAUNCH_CHECK();
        launch(decay_chunk_scan_kernel, dim3((n * nv + 255) / 256, H, n_long), dim3(256), 0, stream, p);
        BG_LAUNCH_CHECK();
        launch(kout, dim3(H, n_chunks), dim3(DC_THREADS), smem_out, stream, p);
    });
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_add_terms_norm(float* x, int n_rows, int d, int assign, int n_terms, const void* const* terms, const int* dtypes,
                                 const int* parts, const long long* part_strides, const float* scales, const void* w1,
                                 const void* w2, int w_dtype, float eps, void* out1, void* out2, int out_dtype,
                                 cudaStream_t stream) {
    if (n_rows <= 0 || d <= 0) return BG_OK;
    if (n_terms < 0 || n_terms > MAX_TERMS || (out2 && !out1) || (out1 && !w1) || (out2 && !w2)) return BG_ERR_SHAPE;
    TermsParams p;
    p.x = x; p.n_terms = n_terms; p.assign = assign; p.w1 = w1; p.w2 = w2; p.w_dtype = w_dtype; p.eps = eps; p.out1 = out1;
    p.out2 = out2; p.out_dtype = out_dtype; p.d = d;
    for (int i = 0; i < MAX_TERMS; ++i) {
        const bool have = i < n_terms;
        p.term[i] = have ? terms[i] : nullptr; p.dtype[i] = have ? dtypes[i] : BG_DTYPE_F32; p.parts[i] = have ? parts[i] : 0;
        p.part_stride[i] = have ? (size_t)part_strides[i] : 0; p.scale[i] = have ? scales[i] : 0.0f;
        if (have && (parts[i] < 1 || (dtypes[i] != BG_DTYPE_F32 && dtypes[i] != BG_DTYPE_BF16))) return BG_ERR_SHAPE;
    }
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    if (smem > BG_SMEM_OPT_IN) {
        cudaError_t e = cudaFuncSetAttribute(add_terms_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(add_terms_norm_vec4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    bool vec = d % 4 == 0 && ((uintptr_t)x % 16) == 0 && (!out1 || (uintptr_t)out1 % 16 == 0) && (!out2 || (uintptr_t)out2 % 16 == 0);
    for (int i = 0; i < n_terms; ++i)
        vec = vec && ((uintptr_t)terms[i] % 16) == 0 && (part_strides[i] % 4) == 0;
    // steps of few rows cannot fill the device with rows: a row's groups of four columns then get a thread each
    const int vthreads = n_rows >= 512 ? 256 : (d / 4 + 31) / 32 * 32 < 64 ? 64 : (d / 4 + 31) / 32 * 32 > 1024 ? 1024 : (d / 4 + 31) / 32 * 32;
    if (vec) launch(add_terms_norm_vec4_kernel, dim3(n_rows), dim3(vthreads), smem, stream, p);
    else launch(add_terms_norm_kernel, dim3(n_rows), dim3(256), smem, stream, p);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
