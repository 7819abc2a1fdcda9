// Linear attention with a constant decay per head, and the sum that joins the branches of a layer.
//
// Per head, with q, k (n features) and v (nv features) of a token, all three silu of a product of the mixer's input:
//     S <- d S + k v^T        (S is n x nv, float, one per request and head, zero when the request starts)
//     o  = S^T q
// The state is carried from step to step in a slot of the cache manager's slab.  Everything is float: the state, the
// decay, the products that enter it and the readout.  Two kernels:
//   decay_attention_seq_kernel    one block per (head, request) walks the request's tokens in turn, the state in shared
//                                 memory.  For steps of single tokens and short portions, and for any sizes.
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
        if (e != cudaSuccess) return (int)e;
    }
    launch(add_terms_norm_kernel, dim3(n_rows), dim3(256), smem, stream, p);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
