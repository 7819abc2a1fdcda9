// What stands between the q/k/v product and the attention for a mixer whose queries and keys are normed over the
// WHOLE projection and whose values may be narrower than its keys: for every token of a step
//   q <- q * rsqrt(mean over all heads' features of q^2 + eps) * wq      (likewise k with wk; skipped without weights)
//   the leading `rot` features of every head of q and k turn by the token's angles (pairs (i, i + rot/2), or
//   (2i, 2i + 1) when interleaved); the rest pass unchanged
//   q goes to q_out [T, nh*hd]; k and v go to the token's place in the paged cache.
// A page holds the keys of all kv heads, [nkv][page_size][hd], followed by their values, [nkv][page_size][vd]; with
// vd == hd that is the layout [2][nkv][page_size][hd] of the other attention kernels.  The heads may be stored wider than
// they are (`qs`, `ks`, `vs` features apart for queries, keys and values, the rest zeros): a head of 96 or of 128 + 32
// features then fills the 64 or 128 that the tensor-core attention kernels take, and a zero adds nothing to a score or
// to a weighted sum.
// The source rows are [q | k | v | ...] as the product left them (any trailing columns are ignored), or the float
// partial sums of a split-K product, added in index order.  Statistics, scaling and rotation are float; a value is
// rounded once, when it is stored.  One block per token, its q and k held in shared memory.
#include <type_traits>

#include "common.cuh"

namespace bg {

struct QkNormRopeParams {
    const void* src; int src_stride; int parts; size_t part_stride;
    void* q_out; int q_stride;
    const float* wq; const float* wk; float eps;            // null: no norm
    int per_head;                                            // 1: every head has a root mean square of its own, and wq, wk hold hd weights
    const float* cos_sin;                                    // [T][rot/2][2] or null when rot == 0
    const int* positions; const int* row_req; const int* block_table; int max_pages;
    void* pool; int num_pages, page_size;                    // null pool: the rows hold queries only
    int nh, nkv, hd, vd, rot, interleaved;
    int qs, ks, vs;                                          // stored width of a query, key and value head (>= hd, hd, vd)
    unsigned* status;
};

// Every head of the staged queries and keys divided by its own root mean square and multiplied by the weights of its
// kind (one vector of hd weights for all query heads, one for all key heads).  A warp per head.
__device__ __forceinline__ void norm_heads_in_place(float* qk_s, const QkNormRopeParams& p, int n_heads) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int h = warp; h < n_heads; h += n_warps) {
        float* v = qk_s + (size_t)h * p.hd;
        const float* w = h < p.nh ? p.wq : p.wk;
        float ss = 0.0f;
        for (int f = lane; f < p.hd; f += 32) ss += v[f] * v[f];
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)p.hd + p.eps);
        for (int f = lane; f < p.hd; f += 32) v[f] = v[f] * inv * w[f];
    }
}

template <typename TS, typename TQ, typename TC>
__global__ void __launch_bounds__(256) qk_norm_rope_append_kernel(QkNormRopeParams p) {
    extern __shared__ float qk_s[];                          // [nh*hd] queries, then [nkv*hd] keys
    __shared__ float red[32];
    pdl_launch();
    const int t = blockIdx.x;
    const int qd = p.nh * p.hd, kd = p.pool ? p.nkv * p.hd : 0, vdd = p.pool ? p.nkv * p.vd : 0;
    const int half = p.rot / 2;
    const TS* row = (const TS*)p.src + (size_t)t * p.src_stride;
    // the token's place depends on no kernel of the step
    const int pos = p.positions[t];
    long long k_base = -1, v_base = -1;
    if (p.pool) {
        const int req = p.row_req[t];
        const int page = p.block_table[(size_t)req * p.max_pages + pos / p.page_size];
        if (page < 0 || page >= p.num_pages) {
            if (p.status && threadIdx.x == 0) atomicOr(p.status, BG_STATUS_BAD_PAGE);
        } else {
            const size_t page_elems = (size_t)p.nkv * p.page_size * (p.ks + p.vs);
            const int slot = pos % p.page_size;
            k_base = (long long)((size_t)page * page_elems + (size_t)slot * p.ks);
            v_base = (long long)((size_t)page * page_elems + (size_t)p.nkv * p.page_size * p.ks + (size_t)slot * p.vs);
        }
    }
    pdl_wait();
    float ssq = 0.0f, ssk = 0.0f;
    for (int i = threadIdx.x; i < qd + kd; i += blockDim.x) {
        const float v = sum_parts(row + i, p.parts, p.part_stride);
        qk_s[i] = v;
        if (i < qd) ssq += v * v; else ssk += v * v;
    }
    if (p.wq && p.per_head) {
        __syncthreads();
        norm_heads_in_place(qk_s, p, p.nh + (p.pool ? p.nkv : 0));
    } else if (p.wq) {
        ssq = block_sum(ssq, red);
        ssk = block_sum(ssk, red);
        const float inv_q = 1.0f / sqrtf(ssq / (float)qd + p.eps);
        const float inv_k = kd > 0 ? 1.0f / sqrtf(ssk / (float)kd + p.eps) : 0.0f;
        __syncthreads();
        for (int i = threadIdx.x; i < qd + kd; i += blockDim.x)
            qk_s[i] = i < qd ? qk_s[i] * inv_q * p.wq[i] : qk_s[i] * inv_k * p.wk[i - qd];
    }
    __syncthreads();
    const float* cs = p.cos_sin ? p.cos_sin + (size_t)t * half * 2 : nullptr;
    TQ* qo = (TQ*)p.q_out + (size_t)t * p.q_stride;
    TC* pool = (TC*)p.pool;
    for (int i = threadIdx.x; i < qd + kd; i += blockDim.x) {
        const int j = i < qd ? i : i - qd;
        const int h = j / p.hd, f = j - h * p.hd;
        float v = qk_s[i];
        if (f < p.rot) {
            int pair, partner;
            bool low;
            if (p.interleaved) { pair = f >> 1; low = (f & 1) == 0; partner = low ? i + 1 : i - 1; }
            else { low = f < half; pair = low ? f : f - half; partner = low ? i + half : i - half; }
            const float c = cs[2 * pair], s = cs[2 * pair + 1], o = qk_s[partner];
            v = low ? v * c - o * s : v * c + o * s;
        }
        if (i < qd) qo[(size_t)h * p.qs + f] = from_float<TQ>(v);
        else if (k_base >= 0) pool[k_base + (size_t)h * p.page_size * p.ks + f] = from_float<TC>(v);
    }
    if (v_base >= 0) {
        for (int i = threadIdx.x; i < vdd; i += blockDim.x) {
            const int h = i / p.vd, f = i - h * p.vd;
            pool[v_base + (size_t)h * p.page_size * p.vs + f] = from_float<TC>(sum_parts(row + qd + kd + i, p.parts, p.part_stride));
        }
    }
    // heads stored wider than they are: zeros behind every head
    const int qpad = p.qs - p.hd, kpad = p.ks - p.hd, vpad = p.vs - p.vd;
    for (int i = threadIdx.x; i < p.nh * qpad; i += blockDim.x) qo[(size_t)(i / qpad) * p.qs + p.hd + i % qpad] = from_float<TQ>(0.0f);
    if (k_base >= 0)
        for (int i = threadIdx.x; i < p.nkv * kpad; i += blockDim.x)
            pool[k_base + (size_t)(i / kpad) * p.page_size * p.ks + p.hd + i % kpad] = from_float<TC>(0.0f);
    if (v_base >= 0)
        for (int i = threadIdx.x; i < p.nkv * vpad; i += blockDim.x)
            pool[v_base + (size_t)(i / vpad) * p.page_size * p.vs + p.vd + i % vpad] = from_float<TC>(0.0f);
}

// The same for sizes in multiples of 8 (heads, stored widths, the rotated part's halves, the source's columns) with the
// rotation in halves or in neighbouring pairs: every access moves eight values, 16 bytes of bfloat16.  A thread's eight
// features lie in one head and, in halves, on one side of the rotated part, so their partners are eight consecutive
// features too; in neighbouring pairs they are four pairs of the thread's own.
template <typename TS, typename TQ, typename TC>
__global__ void __launch_bounds__(256) qk_norm_rope_append_vec8_kernel(QkNormRopeParams p) {
    extern __shared__ float qk_s[];
    __shared__ float red[32];
    pdl_launch();
    const int t = blockIdx.x;
    const int qd = p.nh * p.hd, kd = p.pool ? p.nkv * p.hd : 0, vdd = p.pool ? p.nkv * p.vd : 0;
    const int half = p.rot / 2;
    const TS* row = (const TS*)p.src + (size_t)t * p.src_stride;
    const int pos = p.positions[t];
    long long k_base = -1, v_base = -1;
    if (p.pool) {
        const int req = p.row_req[t];
        const int page = p.block_table[(size_t)req * p.max_pages + pos / p.page_size];
        if (page < 0 || page >= p.num_pages) {
            if (p.status && threadIdx.x == 0) atomicOr(p.status, BG_STATUS_BAD_PAGE);
        } else {
            const size_t page_elems = (size_t)p.nkv * p.page_size * (p.ks + p.vs);
            const int slot = pos % p.page_size;
            k_base = (long long)((size_t)page * page_elems + (size_t)slot * p.ks);
            v_base = (long long)((size_t)page * page_elems + (size_t)p.nkv * p.page_size * p.ks + (size_t)slot * p.vs);
        }
    }
    pdl_wait();
    float ssq = 0.0f, ssk = 0.0f;
    for (int i = threadIdx.x * 8; i < qd + kd; i += blockDim.x * 8) {
        float v[8];
        load8(row + i, v);
        for (int pp = 1; pp < p.parts; ++pp) {
            float u[8];
            load8(row + (size_t)pp * p.part_stride + i, u);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += u[e];
        }
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) { qk_s[i + e] = v[e]; ss += v[e] * v[e]; }
        if (i < qd) ssq += ss; else ssk += ss;
    }
    float inv_q = 1.0f, inv_k = 1.0f;
    const bool whole = p.wq && !p.per_head;                  // the norm over the whole row is applied on the way out
    if (p.wq && p.per_head) {
        __syncthreads();
        norm_heads_in_place(qk_s, p, p.nh + (p.pool ? p.nkv : 0));
    } else if (p.wq) {
        ssq = block_sum(ssq, red);
        ssk = block_sum(ssk, red);
        inv_q = 1.0f / sqrtf(ssq / (float)qd + p.eps);
        inv_k = kd > 0 ? 1.0f / sqrtf(ssk / (float)kd + p.eps) : 0.0f;
    }
    __syncthreads();
    const float* cs = p.cos_sin ? p.cos_sin + (size_t)t * half * 2 : nullptr;
    TQ* qo = (TQ*)p.q_out + (size_t)t * p.q_stride;
    TC* pool = (TC*)p.pool;
    for (int i = threadIdx.x * 8; i < qd + kd; i += blockDim.x * 8) {
        const bool is_q = i < qd;
        const int j = is_q ? i : i - qd;
        const int h = j / p.hd, f = j - h * p.hd;
        const float inv = is_q ? inv_q : inv_k;
        const float* w = whole ? (is_q ? p.wq + j : p.wk + j) : nullptr;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = w ? qk_s[i + e] * inv * w[e] : qk_s[i + e];
        if (f < p.rot && p.interleaved) {
            // neighbouring pairs: the thread's eight features are four pairs of its own, (f + 2k, f + 2k + 1)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = v[2 * k], b = v[2 * k + 1];
                const float c = cs[2 * (f / 2 + k)], sn = cs[2 * (f / 2 + k) + 1];
                v[2 * k] = a * c - b * sn;
                v[2 * k + 1] = b * c + a * sn;
            }
        } else if (f < p.rot) {
            const bool low = f < half;
            const int pair = low ? f : f - half, partner = low ? i + half : i - half;
            const float* wp = w ? (low ? w + half : w - half) : nullptr;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float o = wp ? qk_s[partner + e] * inv * wp[e] : qk_s[partner + e];
                const float c = cs[2 * (pair + e)], sn = cs[2 * (pair + e) + 1];
                v[e] = low ? v[e] * c - o * sn : v[e] * c + o * sn;
            }
        }
        if (is_q) store8(qo + (size_t)h * p.qs + f, v);
        else if (k_base >= 0) store8(pool + k_base + (size_t)h * p.page_size * p.ks + f, v);
    }
    if (v_base >= 0) {
        for (int i = threadIdx.x * 8; i < vdd; i += blockDim.x * 8) {
            const int h = i / p.vd, f = i - h * p.vd;
            float v[8];
            load8(row + qd + kd + i, v);
            for (int pp = 1; pp < p.parts; ++pp) {
                float u[8];
                load8(row + (size_t)pp * p.part_stride + qd + kd + i, u);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += u[e];
            }
            store8(pool + v_base + (size_t)h * p.page_size * p.vs + f, v);
        }
    }
    const float zero[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    const int qpad = (p.qs - p.hd) / 8, kpad = (p.ks - p.hd) / 8, vpad = (p.vs - p.vd) / 8;
    for (int i = threadIdx.x; i < p.nh * qpad; i += blockDim.x) store8(qo + (size_t)(i / qpad) * p.qs + p.hd + 8 * (i % qpad), zero);
    if (k_base >= 0)
        for (int i = threadIdx.x; i < p.nkv * kpad; i += blockDim.x)
            store8(pool + k_base + (size_t)(i / kpad) * p.page_size * p.ks + p.hd + 8 * (i % kpad), zero);
    if (v_base >= 0)
        for (int i = threadIdx.x; i < p.nkv * vpad; i += blockDim.x)
            store8(pool + v_base + (size_t)(i / vpad) * p.page_size * p.vs + p.vd + 8 * (i % vpad), zero);
}

// out[t][j] = src[t][(j / vd) * head_stride + j % vd] * sigmoid(gate[t][col0 + j / gate_per]) for j < n: the gate is a column
// range of a wider row (or of its partial sums), one number per feature (gate_per 1) or one per head (gate_per = vd); the
// source's heads may be stored wider than they are (out == src when they are not).
template <typename TG, typename TO>
__global__ void sigmoid_gate_kernel(TO* __restrict__ out, int out_stride, const TO* __restrict__ src, int src_stride, int vd,
                                    int head_stride, const TG* __restrict__ gate, int gate_stride, int parts,
                                    size_t part_stride, int col0, int rows, int n, int gate_per) {
    pdl_launch();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool idle = idx >= (size_t)rows * n;
    const size_t t = idle ? 0 : idx / n;
    const int j = idle ? 0 : (int)(idx - t * n);
    pdl_wait();
    if (idle) return;
    const float g = sum_parts(gate + t * gate_stride + col0 + j / gate_per, parts, part_stride);
    const float v = to_float(src[t * src_stride + (size_t)(j / vd) * head_stride + j % vd]);
    out[t * out_stride + j] = from_float<TO>(v / (1.0f + expf(-g)));
}

// Eight values a thread (n, vd, the strides and col0 in multiples of 8, everything 16-byte aligned).
template <typename TG, typename TO>
__global__ void sigmoid_gate_vec8_kernel(TO* __restrict__ out, int out_stride, const TO* __restrict__ src, int src_stride, int vd,
                                         int head_stride, const TG* __restrict__ gate, int gate_stride, int parts,
                                         size_t part_stride, int col0, int rows, int n, int gate_per) {
    pdl_launch();
    const int n8 = n >> 3;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool idle = idx >= (size_t)rows * n8;
    const size_t t = idle ? 0 : idx / n8;
    const int j = idle ? 0 : 8 * (int)(idx - t * n8);
    pdl_wait();
    if (idle) return;
    float g[8], v[8];
    if (gate_per > 1) {                       // one gate for the eight values (gate_per is a multiple of 8)
        const float one = sum_parts(gate + t * gate_stride + col0 + j / gate_per, parts, part_stride);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = one;
    } else {
        load8(gate + t * gate_stride + col0 + j, g);
        for (int pp = 1; pp < parts; ++pp) {
            float u[8];
            load8(gate + (size_t)pp * part_stride + t * gate_stride + col0 + j, u);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] += u[e];
        }
    }
    load8(src + t * src_stride + (size_t)(j / vd) * head_stride + j % vd, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fdividef(v[e], 1.0f + __expf(-g[e]));
    store8(out + t * out_stride + j, v);
}

}  // namespace bg

using namespace bg;

template <typename TS, typename TQ, typename TC>
static int qk_norm_rope_launch(const QkNormRopeParams& p, int T, cudaStream_t stream) {
    const int width = p.nh * p.hd + (p.pool ? p.nkv * (p.hd + p.vd) : 0);
    const bool vec = !std::is_same<TQ, float>::value && p.hd % 8 == 0 && p.vd % 8 == 0 && p.rot % (p.interleaved ? 8 : 16) == 0 &&
                     p.qs % 8 == 0 && p.ks % 8 == 0 && p.vs % 8 == 0 && p.src_stride % 8 == 0 && p.part_stride % 8 == 0 &&
                     p.q_stride % 8 == 0 && (uintptr_t)p.src % 16 == 0 && (uintptr_t)p.q_out % 16 == 0 && (uintptr_t)p.pool % 16 == 0 &&
                     (!p.wq || ((uintptr_t)p.wq % 16 == 0 && (uintptr_t)p.wk % 16 == 0)) && width > 0;
    auto kern = vec ? qk_norm_rope_append_vec8_kernel<TS, TQ, TC> : qk_norm_rope_append_kernel<TS, TQ, TC>;
    const size_t smem = (size_t)(p.nh * p.hd + (p.pool ? p.nkv * p.hd : 0)) * sizeof(float);
    if (smem > 200 * 1024) return BG_ERR_SHAPE;
    if (smem > BG_SMEM_OPT_IN) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    launch(kern, dim3(T), dim3(256), smem, stream, p);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_qk_norm_rope_append(const void* src, int src_dtype, int src_stride, int parts, long long part_stride,
                                      void* q_out, int q_dtype, int q_stride, const float* wq, const float* wk, float eps,
                                      const float* cos_sin, const int* positions, const int* row_req, const int* block_table,
                                      int max_pages, void* pool, int cache_dtype, int num_pages, int page_size, int T, int nh,
                                      int nkv, int hd, int vd, int rot, int interleaved, int qs, int ks, int vs, int per_head,
                                      unsigned* status, cudaStream_t stream) {
    if (T <= 0) return BG_OK;
    if (rot < 0 || rot > hd || rot % 2 || parts < 1 || (rot > 0 && !cos_sin) || ((wq == nullptr) != (wk == nullptr))) return BG_ERR_SHAPE;
    if (qs < hd || ks < hd || vs < vd) return BG_ERR_SHAPE;
    if (src_dtype != q_dtype && src_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;
    QkNormRopeParams p;
    p.src = src; p.src_stride = src_stride; p.parts = parts; p.part_stride = (size_t)part_stride; p.q_out = q_out;
    p.q_stride = q_stride; p.wq = wq; p.wk = wk; p.eps = eps; p.cos_sin = cos_sin; p.positions = positions; p.row_req = row_req;
    p.block_table = block_table; p.max_pages = max_pages; p.pool = pool; p.num_pages = num_pages; p.page_size = page_size;
    p.nh = nh; p.nkv = nkv; p.hd = hd; p.vd = vd; p.rot = rot; p.interleaved = interleaved; p.qs = qs; p.ks = ks; p.vs = vs; p.per_head = per_head; p.status = status;
    if (!pool) cache_dtype = q_dtype;
    if (cache_dtype != q_dtype) return BG_ERR_DTYPE;            // queries and cache are both of the compute type
    if (q_dtype == BG_DTYPE_F32) {
        if (src_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;
        return qk_norm_rope_launch<float, float, float>(p, T, stream);
    }
    if (src_dtype == BG_DTYPE_F32) return qk_norm_rope_launch<float, __nv_bfloat16, __nv_bfloat16>(p, T, stream);
    return qk_norm_rope_launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(p, T, stream);
}

extern "C" int bg_sigmoid_gate(void* out, int out_dtype, int out_stride, const void* src, int src_stride, int vd, int head_stride,
                               const void* gate, int gate_dtype, int gate_stride, int parts, long long part_stride, int col0,
                               int rows, int n, int gate_per, cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return BG_OK;
    if (parts < 1 || vd <= 0 || head_stride < vd || gate_per < 1) return BG_ERR_SHAPE;
    const size_t total = (size_t)rows * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    const bool vec = out_dtype == BG_DTYPE_BF16 && n % 8 == 0 && vd % 8 == 0 && head_stride % 8 == 0 && out_stride % 8 == 0 &&
                     src_stride % 8 == 0 && (gate_per > 1 ? gate_per % 8 == 0 : (gate_stride % 8 == 0 && col0 % 8 == 0 && part_stride % 8 == 0)) &&
                     (uintptr_t)out % 16 == 0 && (uintptr_t)src % 16 == 0 && (gate_per > 1 || (uintptr_t)gate % 16 == 0);
    if (vec) {
        const unsigned vblocks = (unsigned)((total / 8 + 255) / 256);
        BG_DISPATCH_DTYPE(gate_dtype, TG,
            launch(sigmoid_gate_vec8_kernel<TG, __nv_bfloat16>, dim3(vblocks), dim3(256), 0, stream, (__nv_bfloat16*)out, out_stride,
                   (const __nv_bfloat16*)src, src_stride, vd, head_stride, (const TG*)gate, gate_stride, parts, (size_t)part_stride,
                   col0, rows, n, gate_per));
        BG_LAUNCH_CHECK();
        return BG_OK;
    }
    BG_DISPATCH_DTYPE(gate_dtype, TG, BG_DISPATCH_DTYPE(out_dtype, TO,
        launch(sigmoid_gate_kernel<TG, TO>, dim3(blocks), dim3(256), 0, stream, (TO*)out, out_stride, (const TO*)src, src_stride, vd,
               head_stride, (const TG*)gate, gate_stride, parts, (size_t)part_stride, col0, rows, n, gate_per)));
    BG_LAUNCH_CHECK();
    return BG_OK;
}
