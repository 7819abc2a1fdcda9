// Routed experts: what stands around the experts' products.
//
//   route_topk     per token, the `top` experts of largest score (score = sigmoid of the router's float logit, or the
//                  logit itself), ties to the lower index; the logits are what is compared, since sigmoid keeps their
//                  order but rounds large ones to equal scores.  The weight of a choice is its score, divided by the
//                  sum of the chosen scores when `renorm`.
//   route_sort     the step's assignments (token t, rank j) -> a = t * top + j are laid out expert by expert:
//                  offsets[e] .. offsets[e + 1] are expert e's rows; row_of[a] is where assignment a went and
//                  src_of[row] the assignment that row holds.  ONE CTA; the order inside an expert is whatever the
//                  atomics give, which no result depends on (a row's product is a function of that row alone).
//   route_gather   xp[row] = (weight * x[token]) rounded to the compute type (or x[token] as it is).
//   gemm_grouped   yp[row] = act(xp[row] W[e]^T) on CUDA cores, float accumulation, every output summed over k in index
//                  order by one thread: the float32 path, and the sizes the tensor-core product does not take.
//   route_combine  out[t] = sum_j (weight *) yp[row_of[t * top + j]], ranks added in index order, float.
//
// Nothing here is read back to the host: the grids depend on the step's shapes alone (the grouped products are launched
// with as many row tiles as any distribution of the tokens could need, and a CTA without rows returns), so a step with
// routed experts can be captured in a graph.
#include "common.cuh"

namespace bg {

// How the router's logits become scores (`mode`): 0 the logit itself, 1 its sigmoid, 2 the softmax over all E logits.
struct RouteRule {
    int mode;
    int renorm;             // the chosen scores are divided by their sum
    const float* bias;      // [E] or null: added to the scores for the CHOICE only; the weights are the scores without it
    float scale;            // multiplies the weights
};

// One warp chooses for one token: `sc` holds the token's E logits in shared memory and is used up.  Without a bias and
// without the softmax the choice is made on the logits: sigmoid keeps their order, but rounds large ones to the same
// score.  Otherwise it is made on score + bias, the scores formed anew from the logits each time; a logit of -inf marks
// an expert that is taken.  Ties go to the lower index.
__device__ __forceinline__ void choose_experts(float* sc, int E, int top, RouteRule rule, int* __restrict__ ids,
                                               float* __restrict__ weights, size_t t, int lane) {
    float total = 0.0f;
    float zmax = 0.0f, inv = 1.0f;
    if (rule.mode == 2) {                                  // softmax over all experts, float
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, sc[e]);
        zmax = warp_max(m);
        float s = 0.0f;
        for (int e = lane; e < E; e += 32) s += expf(sc[e] - zmax);
        inv = 1.0f / warp_sum(s);
    }
    const bool on_scores = rule.mode == 2 || rule.bias != nullptr;
    auto score_of = [&](float z) {
        return rule.mode == 2 ? expf(z - zmax) * inv : (rule.mode == 1 ? 1.0f / (1.0f + expf(-z)) : z);
    };
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            float v = sc[e];
            if (on_scores && v != -INFINITY) v = score_of(v) + (rule.bias ? rule.bias[e] : 0.0f);
            if (v > best) { best = v; arg = e; }            // ascending e: the first of equal scores stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;                     // (every score NaN or -inf: a defined choice)
        const float score = score_of(on_scores ? sc[arg] : best);
        __syncwarp();
        if (lane == 0) {
            ids[(size_t)t * top + j] = arg;
            weights[(size_t)t * top + j] = score * rule.scale;
            sc[arg] = -INFINITY;
        }
        total += score;
        __syncwarp();
    }
    if (rule.renorm && lane < top) weights[(size_t)t * top + lane] /= total;
}

__global__ void route_topk_kernel(const float* __restrict__ logits, int T, int E, int top, RouteRule rule,
                                  int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float score_s[];                     // [warps][E]
    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* sc = score_s + (size_t)warp * E;
    for (int e = lane; e < E; e += 32) sc[e] = logits[(size_t)t * E + e];
    __syncwarp();
    choose_experts(sc, E, top, rule, ids, weights, (size_t)t, lane);
}

// The router of a step in one kernel: a block takes ROUTE_TOKENS tokens; each of its warps takes experts in turn and
// forms the float logits of all the block's tokens against that expert's row (the row is read once per block; a lane
// walks the features 32 apart and the warp adds up, so a logit's order of summation depends on nothing but the width);
// then warp w chooses for token w.  `logits_out`, when given, also receives the logits.
constexpr int ROUTE_TOKENS = 8, ROUTE_UNROLL = 8;
template <typename TI>
__global__ void __launch_bounds__(32 * ROUTE_TOKENS)
route_kernel(const TI* __restrict__ h, int ldh, const float* __restrict__ W, int T, int d, int E, int top, RouteRule rule,
             int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ logits_out) {
    extern __shared__ float logit_s[];                     // [ROUTE_TOKENS][E]
    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * ROUTE_TOKENS;
    const int n = min(ROUTE_TOKENS, T - t0);
    for (int e = warp; e < E; e += ROUTE_TOKENS) {
        float acc[ROUTE_TOKENS];
#pragma unroll
        for (int j = 0; j < ROUTE_TOKENS; ++j) acc[j] = 0.0f;
        const float* w = W + (size_t)e * d;
        // ROUTE_UNROLL features a lane at a time: all their loads go out before the first product (one feature at a time
        // cost a trip to memory per feature: 58 us for 1,536 features, whatever the number of tokens)
        for (int k0 = lane; k0 < d; k0 += 32 * ROUTE_UNROLL) {
            float wk[ROUTE_UNROLL], hv[ROUTE_UNROLL][ROUTE_TOKENS];
#pragma unroll
            for (int u = 0; u < ROUTE_UNROLL; ++u) {
                const int k = k0 + 32 * u;
                wk[u] = k < d ? w[k] : 0.0f;
#pragma unroll
                for (int j = 0; j < ROUTE_TOKENS; ++j)
                    hv[u][j] = (k < d && j < n) ? to_float(h[(size_t)(t0 + j) * ldh + k]) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < ROUTE_UNROLL; ++u)
#pragma unroll
                for (int j = 0; j < ROUTE_TOKENS; ++j) acc[j] = fmaf(hv[u][j], wk[u], acc[j]);
        }
#pragma unroll
        for (int j = 0; j < ROUTE_TOKENS; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0 && j < n) {
                logit_s[j * E + e] = v;
                if (logits_out) logits_out[(size_t)(t0 + j) * E + e] = v;
            }
        }
    }
    __syncthreads();
    if (warp < n) choose_experts(logit_s + warp * E, E, top, rule, ids, weights, (size_t)(t0 + warp), lane);
}

// The same for a width that is a multiple of 8 and 16-byte aligned rows.  A block of eight warps takes TPB tokens, 8 / TPB
// warps to a token, which share the experts in groups of G; a lane walks the token's features in chunks of eight, 32 chunks
// apart (16-byte loads: one of the token's row, which stays in the first-level cache from expert to expert, and two of
// each expert's row), and the warp adds up; the first warp of a token then chooses.  Steps of many tokens: a warp per token,
// four experts at a time.  Steps of few tokens: a block per token and an expert per warp at a time, so that a decoding step
// spreads over as many SMs as it has tokens and a warp's chain of loads is one expert long.  (The walk through the features
// one at a time above cost 53 us for 1,536 features whatever the number of tokens.)
template <typename TI, int TPB, int G>
__global__ void __launch_bounds__(32 * ROUTE_TOKENS)
route_vec8_kernel(const TI* __restrict__ h, int ldh, const float* __restrict__ W, int T, int d, int E, int top, RouteRule rule,
                  int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ logits_out) {
    constexpr int WPT = ROUTE_TOKENS / TPB;                // warps per token
    extern __shared__ float logit_s[];                     // [TPB][E]
    pdl_launch();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tl = warp / WPT, wq = warp % WPT;
    const int t = blockIdx.x * TPB + tl;
    const bool live = t < T;
    const TI* row = h + (size_t)(live ? t : 0) * ldh;
    float* sc = logit_s + tl * E;
    const int d8 = d >> 3;
    for (int e0 = wq * G; live && e0 < E; e0 += WPT * G) {
        float acc[G];
#pragma unroll
        for (int u = 0; u < G; ++u) acc[u] = 0.0f;
#pragma unroll 2
        for (int c = lane; c < d8; c += 32) {
            float hv[8];
            load8(row + 8 * c, hv);
#pragma unroll
            for (int u = 0; u < G; ++u) {
                if (e0 + u < E) {
                    float wv[8];
                    load8(W + (size_t)(e0 + u) * d + 8 * c, wv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[u] = fmaf(hv[i], wv[i], acc[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < G; ++u) {
            const float v = warp_sum(acc[u]);
            if (lane == 0 && e0 + u < E) {
                sc[e0 + u] = v;
                if (logits_out) logits_out[(size_t)t * E + e0 + u] = v;
            }
        }
    }
    __syncthreads();                                       // every warp comes here, with or without a token
    if (live && wq == 0) choose_experts(sc, E, top, rule, ids, weights, (size_t)t, lane);
}

__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ ids, int A, int E, int* __restrict__ offsets, int* __restrict__ row_of,
                  int* __restrict__ src_of) {
    extern __shared__ int count_s[];                       // [E] counts, then [E] cursors
    int* cursor_s = count_s + E;
    pdl_launch();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count_s[e] = 0;
    pdl_wait();
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = ids[a];
        if (e >= 0 && e < E) atomicAdd(&count_s[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { offsets[e] = run; cursor_s[e] = run; run += count_s[e]; }
        offsets[E] = run;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const int e = ids[a];
        if (e < 0 || e >= E) continue;
        const int row = atomicAdd(&cursor_s[e], 1);
        row_of[a] = row;
        src_of[row] = a;
    }
}

template <typename TI, typename TO>
__global__ void route_gather_kernel(const TI* __restrict__ x, const float* __restrict__ weights, const int* __restrict__ src_of,
                                    TO* __restrict__ xp, int A, int d, int top, int scale) {
    pdl_launch();
    pdl_wait();
    const int row = blockIdx.x;
    const int a = src_of[row];
    const float w = scale ? weights[a] : 1.0f;
    const TI* src = x + (size_t)(a / top) * d;
    TO* dst = xp + (size_t)row * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<TO>(w * to_float(src[i]));
}

template <typename TY>
__global__ void route_combine_kernel(const TY* __restrict__ yp, const float* __restrict__ weights, const int* __restrict__ row_of,
                                     float* __restrict__ out, int T, int d, int top, int scale) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int a = t * top + j;
            const float v = to_float(yp[(size_t)row_of[a] * d + i]);
            acc += scale ? weights[a] * v : v;
        }
        out[(size_t)t * d + i] = acc;
    }
}

// The same sum for a layer that also has experts without weights and a shared expert:
//   out[t] = sum_j w_j (id_j < n_real ? yp[row_of[t top + j]] : h[t])  +  sigmoid(sg[t]) shared[t].
// An expert whose index is n_real or more returns its input (the step's rows h in the compute type).  `shared` [T][d]
// float is the result of an expert that every token passes, `sg` one number per token (element t at sg[t * sg_stride], float
// or bfloat16), whose sigmoid multiplies it; without `sg` the shared result is added as it is.  Ranks in index order, float.
template <typename TY, typename TH>
__global__ void route_combine_ext_kernel(const TY* __restrict__ yp, const float* __restrict__ weights, const int* __restrict__ row_of,
                                         const int* __restrict__ ids, int n_real, const TH* __restrict__ h, int ldh,
                                         const float* __restrict__ shared, const void* __restrict__ sg, int sg_float, int sg_stride,
                                         float* __restrict__ out, int T, int d, int top) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    float sgate = shared ? 1.0f : 0.0f;
    if (shared && sg) {
        const float z = sg_float ? ((const float*)sg)[(size_t)t * sg_stride] : __bfloat162float(((const __nv_bfloat16*)sg)[(size_t)t * sg_stride]);
        sgate = 1.0f / (1.0f + expf(-z));
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int a = t * top + j;
            const float v = ids[a] < n_real ? to_float(yp[(size_t)row_of[a] * d + i]) : to_float(h[(size_t)t * ldh + i]);
            acc = fmaf(weights[a], v, acc);
        }
        if (shared) acc = fmaf(sgate, shared[(size_t)t * d + i], acc);
        out[(size_t)t * d + i] = acc;
    }
}

// The same, four columns a thread (d a multiple of 4, float results of the experts, 16-byte aligned rows).
template <typename TH>
__global__ void route_combine_ext_vec4_kernel(const float* __restrict__ yp, const float* __restrict__ weights,
                                              const int* __restrict__ row_of, const int* __restrict__ ids, int n_real,
                                              const TH* __restrict__ h, int ldh, const float* __restrict__ shared,
                                              const void* __restrict__ sg, int sg_float, int sg_stride, float* __restrict__ out, int T,
                                              int d, int top) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    float sgate = shared ? 1.0f : 0.0f;
    if (shared && sg) {
        const float z = sg_float ? ((const float*)sg)[(size_t)t * sg_stride] : __bfloat162float(((const __nv_bfloat16*)sg)[(size_t)t * sg_stride]);
        sgate = 1.0f / (1.0f + expf(-z));
    }
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float4 hv;
        {
            const TH* hp = h + (size_t)t * ldh + i;
            hv = make_float4(to_float(hp[0]), to_float(hp[1]), to_float(hp[2]), to_float(hp[3]));
        }
        for (int j = 0; j < top; ++j) {
            const int a = t * top + j;
            const float w = weights[a];
            const float4 v = ids[a] < n_real ? *reinterpret_cast<const float4*>(yp + (size_t)row_of[a] * d + i) : hv;
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        if (shared) {
            const float4 s = *reinterpret_cast<const float4*>(shared + (size_t)t * d + i);
            acc.x = fmaf(sgate, s.x, acc.x); acc.y = fmaf(sgate, s.y, acc.y); acc.z = fmaf(sgate, s.z, acc.z); acc.w = fmaf(sgate, s.w, acc.w);
        }
        *reinterpret_cast<float4*>(out + (size_t)t * d + i) = acc;
    }
}

// A gated expert's activation with clamps: from a row [gate (n) | up (n)] of the product,
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g sigmoid(alpha g) (u + 1).
// Float arithmetic; the input in either type with `ld` elements between rows, the output contiguous.
template <typename TI, typename TO>
__global__ void glu_clamped_kernel(const TI* __restrict__ gu, int ld, TO* __restrict__ out, size_t total, int n, float limit,
                                   float alpha) {
    pdl_launch();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t r = idx / n;
    const int i = (int)(idx - r * n);
    const float g = fminf(to_float(gu[r * ld + i]), limit);
    const float u = fminf(fmaxf(to_float(gu[r * ld + n + i]), -limit), limit);
    out[idx] = from_float<TO>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

// The same, eight columns a thread (n and ld multiples of 8, 16-byte aligned rows).
template <typename TI, typename TO>
__global__ void glu_clamped_vec8_kernel(const TI* __restrict__ gu, int ld, TO* __restrict__ out, size_t total8, int n, float limit,
                                        float alpha) {
    pdl_launch();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const int n8 = n >> 3;
    const size_t r = idx / n8;
    const int i = (int)(idx - r * n8) * 8;
    float g[8], u[8];
    load8(gu + r * ld + i, g);
    load8(gu + r * ld + n + i, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float gg = fminf(g[e], limit);
        const float uu = fminf(fmaxf(u[e], -limit), limit);
        g[e] = gg / (1.0f + expf(-alpha * gg)) * (uu + 1.0f);
    }
    store8(out + r * n + i, g);
}

// ------------------------------------------------------------------------------------------------ grouped product
// The expert and the rows of row tile `tile` (tiles of `bm` rows, expert after expert); false when there is none.
__device__ __forceinline__ bool group_tile(const int* offsets, int E, int bm, int tile, int* e_out, int* row0, int* n_rows) {
    int before = 0;
    for (int e = 0; e < E; ++e) {
        const int lo = offsets[e], n = offsets[e + 1] - lo;
        const int tiles = (n + bm - 1) / bm;
        if (tile < before + tiles) {
            const int r = (tile - before) * bm;
            *e_out = e; *row0 = lo + r; *n_rows = min(bm, n - r);
            return true;
        }
        before += tiles;
    }
    return false;
}

constexpr int GG_BM = 32, GG_BN = 64, GG_BK = 16, GG_THREADS = 256;

// C[row, n] = act(sum_k A[row, k] W[e][n, k]); ACT 1: the square of relu.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(GG_THREADS)
gemm_grouped_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw, long long w_expert, TC* __restrict__ C,
                    int ldc, const int* __restrict__ offsets, int E, int N, int K, int act) {
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[GG_BK][GG_BN + 4];
    __shared__ int where[3];
    pdl_launch();
    pdl_wait();
    if (threadIdx.x == 0) {
        int e = -1, r0 = 0, n = 0;
        if (!group_tile(offsets, E, GG_BM, blockIdx.y, &e, &r0, &n)) e = -1;
        where[0] = e; where[1] = r0; where[2] = n;
    }
    __syncthreads();
    const int e = where[0], row0 = where[1], n_rows = where[2];
    if (e < 0) return;
    W += (size_t)e * w_expert;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * GG_BN;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, each 2 rows x 4 columns of C
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        // A tile: 32 rows x 16 k = 512 values, two a thread; W tile: 64 rows x 16 k = 1024 values, four a thread
        for (int idx = tid; idx < GG_BM * GG_BK; idx += GG_THREADS) {
            const int r = idx / GG_BK, k = idx - r * GG_BK;
            As[k][r] = (r < n_rows && k0 + k < K) ? to_float(A[(size_t)(row0 + r) * lda + k0 + k]) : 0.0f;
        }
        for (int idx = tid; idx < GG_BN * GG_BK; idx += GG_THREADS) {
            const int r = idx / GG_BK, k = idx - r * GG_BK;
            Ws[k][r] = (n0 + r < N && k0 + k < K) ? to_float(W[(size_t)(n0 + r) * ldw + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[2], w[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (act == 1) { v = fmaxf(v, 0.0f); v *= v; }
            C[(size_t)(row0 + r) * ldc + n] = from_float<TC>(v);
        }
    }
}

// C[M, N] = A[M, K] W[N, K]^T with A of either type and float W and C: the router's logits, float from a step's rows
// in the compute type.  Every output is summed over k in index order by one thread.
template <typename TA>
__global__ void __launch_bounds__(256)
gemm_rows_f32w_kernel(const TA* __restrict__ A, int lda, const float* __restrict__ W, int ldw, float* __restrict__ C, int ldc,
                      int M, int N, int K) {
    __shared__ float As[16][64 + 4];
    __shared__ float Ws[16][64 + 4];
    pdl_launch();
    pdl_wait();
    const int tid = threadIdx.x, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int idx = tid; idx < 64 * 16; idx += 256) {
            const int r = idx >> 4, k = idx & 15;
            As[k][r] = (m0 + r < M && k0 + k < K) ? to_float(A[(size_t)(m0 + r) * lda + k0 + k]) : 0.0f;
            Ws[k][r] = (n0 + r < N && k0 + k < K) ? W[(size_t)(n0 + r) * ldw + k0 + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
}

}  // namespace bg

using namespace bg;

extern "C" int bg_route_logits(const void* A, int a_dtype, int lda, const float* W, int ldw, float* C, int ldc, int M, int N,
                               int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BG_OK;
    if (K <= 0) return BG_ERR_SHAPE;
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (grid.y > 65535) return BG_ERR_SHAPE;
    BG_DISPATCH_DTYPE(a_dtype, TA, launch(gemm_rows_f32w_kernel<TA>, grid, dim3(256), 0, stream, (const TA*)A, lda, W, ldw, C, ldc,
                                          M, N, K));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_route_topk(const float* logits, int T, int E, int top, int mode, int renorm, const float* bias, float scale,
                             int* ids, float* weights, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (E <= 0 || top <= 0 || top > E || top > 32 || mode < 0 || mode > 2) return BG_ERR_SHAPE;
    const RouteRule rule = {mode, renorm, bias, scale};
    const int warps = 4;
    const size_t smem = (size_t)warps * E * sizeof(float);
    if (smem > 40 * 1024) return BG_ERR_UNSUPPORTED;
    launch(route_topk_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), smem, stream, logits, T, E, top, rule, ids,
           weights);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// The router in one kernel: float logits of h [T, d] (either type, row stride ldh) against W [E, d] float, and the choice.
extern "C" int bg_route(const void* h, int h_dtype, int ldh, const float* W, int T, int d, int E, int top, int mode, int renorm,
                        const float* bias, float scale, int* ids, float* weights, float* logits_out, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (E <= 0 || top <= 0 || top > E || top > 32 || d <= 0 || mode < 0 || mode > 2) return BG_ERR_SHAPE;
    const RouteRule rule = {mode, renorm, bias, scale};
    const size_t smem = (size_t)ROUTE_TOKENS * E * sizeof(float);
    if (smem > 40 * 1024) return BG_ERR_UNSUPPORTED;
    const dim3 grid((T + ROUTE_TOKENS - 1) / ROUTE_TOKENS), block(32 * ROUTE_TOKENS);
    // experts a warp takes at a time in steps of few tokens: as many as let a token's experts go through in one pass (the loads
    // of a pass are all on their way together; every expert's sum keeps its own order, so the logits are the same bits: 9.3 ->
    // 7.8 us for ten router outputs)
    const bool vec = d % 8 == 0 && ldh % 8 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)W % 16 == 0;
#define BG_ROUTE_VEC(TPB, G, GRID, SMEM)                                                                                \
    BG_DISPATCH_DTYPE(h_dtype, TI, launch(route_vec8_kernel<TI, TPB, G>, GRID, block, SMEM, stream, (const TI*)h, ldh, W, T, d, E, \
                                          top, rule, ids, weights, logits_out))
    if (vec && T <= 256) {
        const size_t one = (size_t)E * sizeof(float);
        if (E <= ROUTE_TOKENS) BG_ROUTE_VEC(1, 1, dim3(T), one);
        else if (E <= 2 * ROUTE_TOKENS) BG_ROUTE_VEC(1, 2, dim3(T), one);
        else BG_ROUTE_VEC(1, 4, dim3(T), one);
    } else if (vec) {
        BG_ROUTE_VEC(ROUTE_TOKENS, 4, grid, smem);     // (sixteen at a time: 39.7 against 25.3 us for 2,048 tokens and ten experts)
    } else
#undef BG_ROUTE_VEC
        BG_DISPATCH_DTYPE(h_dtype, TI, launch(route_kernel<TI>, grid, block, smem, stream, (const TI*)h, ldh, W, T, d, E, top, rule,
                                              ids, weights, logits_out));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_route_sort(const int* ids, int A, int E, int* offsets, int* row_of, int* src_of, cudaStream_t stream) {
    if (E <= 0 || A < 0) return BG_ERR_SHAPE;
    const size_t smem = (size_t)2 * E * sizeof(int);
    if (smem > 40 * 1024) return BG_ERR_UNSUPPORTED;
    launch(route_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, A, E, offsets, row_of, src_of);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_route_gather(const void* x, int x_dtype, const float* weights, const int* src_of, void* xp, int xp_dtype, int A,
                               int d, int top, int scale, cudaStream_t stream) {
    if (A <= 0) return BG_OK;
    const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
    BG_DISPATCH_DTYPE(x_dtype, TI, BG_DISPATCH_DTYPE(xp_dtype, TO,
        launch(route_gather_kernel<TI, TO>, dim3(A), dim3(threads), 0, stream, (const TI*)x, weights, src_of, (TO*)xp, A, d, top, scale)));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_route_combine(const void* yp, int y_dtype, const float* weights, const int* row_of, float* out, int T, int d,
                                int top, int scale, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
    BG_DISPATCH_DTYPE(y_dtype, TY, launch(route_combine_kernel<TY>, dim3(T), dim3(threads), 0, stream, (const TY*)yp, weights, row_of,
                                          out, T, d, top, scale));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_route_combine_ext(const void* yp, int y_dtype, const float* weights, const int* row_of, const int* ids, int n_real,
                                    const void* h, int h_dtype, int ldh, const float* shared, const void* sg, int sg_dtype,
                                    int sg_stride, float* out, int T, int d, int top, cudaStream_t stream) {
    const int sg_float = sg_dtype == BG_DTYPE_F32 ? 1 : 0;
    if (T <= 0) return BG_OK;
    if (!ids || !h || top <= 0) return BG_ERR_SHAPE;
    const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
    if (y_dtype == BG_DTYPE_F32 && d % 4 == 0 && ldh % 4 == 0 && (uintptr_t)yp % 16 == 0 && (uintptr_t)out % 16 == 0 &&
        (!shared || (uintptr_t)shared % 16 == 0)) {
        const int tv = d / 4 >= 384 ? 384 : ((d / 4 + 31) / 32) * 32;
        BG_DISPATCH_DTYPE(h_dtype, TH, launch(route_combine_ext_vec4_kernel<TH>, dim3(T), dim3(tv), 0, stream, (const float*)yp, weights,
                                              row_of, ids, n_real, (const TH*)h, ldh, shared, sg, sg_float, sg_stride, out, T, d, top));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    BG_DISPATCH_DTYPE(y_dtype, TY, BG_DISPATCH_DTYPE(h_dtype, TH,
        launch(route_combine_ext_kernel<TY, TH>, dim3(T), dim3(threads), 0, stream, (const TY*)yp, weights, row_of, ids, n_real,
               (const TH*)h, ldh, shared, sg, sg_float, sg_stride, out, T, d, top)));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_glu_clamped(const void* gu, int gu_dtype, int ld, void* out, int out_dtype, int rows, int n, float limit,
                              float alpha, cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return BG_OK;
    if (ld < 2 * n) return BG_ERR_SHAPE;
    const size_t total = (size_t)rows * n;
    if ((total + 255) / 256 > 0x7fffffffULL) return BG_ERR_SHAPE;
    if (n % 8 == 0 && ld % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t total8 = total / 8;
        BG_DISPATCH_DTYPE(gu_dtype, TI, BG_DISPATCH_DTYPE(out_dtype, TO,
            launch(glu_clamped_vec8_kernel<TI, TO>, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, stream, (const TI*)gu, ld,
                   (TO*)out, total8, n, limit, alpha)));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    BG_DISPATCH_DTYPE(gu_dtype, TI, BG_DISPATCH_DTYPE(out_dtype, TO,
        launch(glu_clamped_kernel<TI, TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const TI*)gu, ld, (TO*)out,
               total, n, limit, alpha)));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

// A [rows, K] (float or bfloat16), W [E][N, K] of the same type with w_expert elements between experts, C [rows, N] float or of
// A's type.  `rows` is the number of assignments: the grid has a row tile for every tile any distribution could need.
extern "C" int bg_gemm_grouped(const void* A, int a_dtype, int lda, const void* W, int ldw, long long w_expert, void* C, int c_dtype,
                               int ldc, const int* offsets, int E, int rows, int N, int K, int act, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return BG_OK;
    if (K <= 0 || E <= 0) return BG_ERR_SHAPE;
    const int row_tiles = rows / GG_BM + E;
    if (row_tiles > 65535) return BG_ERR_SHAPE;
    dim3 grid((N + GG_BN - 1) / GG_BN, row_tiles);
    if (a_dtype == BG_DTYPE_F32 && c_dtype == BG_DTYPE_F32)
        launch(gemm_grouped_kernel<float, float, float>, grid, dim3(GG_THREADS), 0, stream, (const float*)A, lda, (const float*)W, ldw,
               w_expert, (float*)C, ldc, offsets, E, N, K, act);
    else if (a_dtype == BG_DTYPE_BF16 && c_dtype == BG_DTYPE_BF16)
        launch(gemm_grouped_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, dim3(GG_THREADS), 0, stream,
               (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, w_expert, (__nv_bfloat16*)C, ldc, offsets, E, N, K, act);
    else if (a_dtype == BG_DTYPE_BF16 && c_dtype == BG_DTYPE_F32)
        launch(gemm_grouped_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, dim3(GG_THREADS), 0, stream,
               (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, w_expert, (float*)C, ldc, offsets, E, N, K, act);
    else return BG_ERR_DTYPE;
    BG_LAUNCH_CHECK();
    return BG_OK;
}
