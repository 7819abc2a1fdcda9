// Attention through a low-rank latent, over a paged cache that holds, per position, ONE row for all
// heads: the normed latent c [rank] followed by the rotated key part k_r [rot] that the heads share.
//
// The per-head keys W_uk c and values W_uv c are never made.  With a = W_uk^T q_plain (the query
// carried into the latent space, a product that the caller runs per head), the score of a key is
//   s_t = (a . c_t + q_rot . k_r,t) * scale,
// and with the softmax weights p the head's result in the latent space is o = sum_t p_t c_t, from which
// the caller makes W_uv o.  So every head attends over the same cached rows: the first `rank` features
// of a row serve as its value.
//
// The layout of the work is that of the grouped-query kernel (attention.cu): query blocks of up to `bq`
// consecutive rows of one request, keys cut into splits at absolute positions, one CTA per (query block,
// chunk of heads, split) that streams its keys once for all its rows and writes, per (row, head), a
// running maximum, a running sum and an unnormalised result; a merge kernel joins the splits in order.
// Everything is float, and a row shares no accumulator with another row, so a row's result does not
// depend on how the step was cut or on what else is in the batch.
#include "common.cuh"

namespace bg {

constexpr int LAT_THREADS = 256;
constexpr int LAT_WARPS = LAT_THREADS / 32;

// One block per step row: the RMS norm of the latent and the rotation of the shared key part, stored at the
// row's position in the pages.  src row = [.. | latent raw (rank) | key part raw (rot) | ..] from col0.
// Pairs (2i, 2i+1) of the first rot_dims features of the key part turn by the row's angles; the rest pass.
// With q_out, the same block also norms the row's query latent src[q_col0 .. q_col0 + q_rank) into q_out[t]
// (the two norms read the same product's row, so they share a launch).
template <typename TI, typename TW, typename TC, typename TQ>
__global__ void latent_append_kernel(const TI* __restrict__ src, int src_stride, int col0, int rank, int rot, int rot_dims,
                                     const TW* __restrict__ w, float eps, const float* __restrict__ cos_sin,
                                     const int* __restrict__ positions, const int* __restrict__ row_req,
                                     const int* __restrict__ block_table, int max_pages, TC* __restrict__ pool,
                                     int num_pages, int page_size, unsigned* status, int q_col0, int q_rank,
                                     const TW* __restrict__ q_w, TQ* __restrict__ q_out) {
    __shared__ float red[32];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    if (q_out) {
        const TI* qs = src + (size_t)t * src_stride + q_col0;
        float qq = 0.0f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_float(qs[i]);
            qq += v * v;
        }
        qq = block_sum(qq, red);
        const float qinv = 1.0f / sqrtf(qq / (float)q_rank + eps);
        TQ* qo = q_out + (size_t)t * q_rank;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) qo[i] = from_float<TQ>(to_float(qs[i]) * qinv * to_float(q_w[i]));
    }
    const TI* s = src + (size_t)t * src_stride + col0;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(s[i]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)row_req[t] * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicOr(status, BG_STATUS_BAD_PAGE);
        return;
    }
    const int width = rank + rot;
    TC* dst = pool + ((size_t)page * page_size + pos % page_size) * width;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<TC>(to_float(s[i]) * inv * to_float(w[i]));
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = to_float(s[rank + 2 * i]), v = to_float(s[rank + 2 * i + 1]);
        const float c = cos_sin[((size_t)t * half + i) * 2], sn = cos_sin[((size_t)t * half + i) * 2 + 1];
        dst[rank + 2 * i] = from_float<TC>(u * c - v * sn);
        dst[rank + 2 * i + 1] = from_float<TC>(v * c + u * sn);
    }
    for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = from_float<TC>(to_float(s[rank + i]));
}

struct LatentParams {
    const void* q_lat;      // [H][T][rank] queries in the latent space: element (h, t, i) at h*ql_head + t*ql_row + i
    long long ql_head;
    int ql_row;
    const void* q_raw;      // [T][H][dim + rot] the query product's rows: the rot part of head h starts at h*(dim+rot) + dim
    int qr_row, qr_head, qr_off;
    const float* cos_sin;   // [T][rot_dims/2][2]
    const void* pool;       // [num_pages][page_size][rank + rot]
    int num_pages, page_size;
    const int* block_table; // [B, max_pages]
    int max_pages;
    const int* positions;   // [T]
    const int* qblk;        // [n_qblk][3] = (request, first row, number of rows)
    float* part_o;          // [T*H][max_splits][rank]
    float* part_ml;         // [T*H][max_splits][2]
    int max_splits;
    int H, hc;              // heads, heads per CTA
    int rank, rot, rot_dims;
    int split, tile, bq;
    int window;             // as first_visible() reads it; 0: every earlier position
    float scale;
    unsigned* status;
};

template <typename TQ, typename TR, typename TC>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_partial_kernel(LatentParams p) {
    extern __shared__ float smem[];
    const int rank = p.rank, width = p.rank + p.rot;
    const int kstride = width + 1;
    const int rows_max = p.bq * p.hc;
    float* q_s = smem;                                       // [rows_max][width]
    float* acc_s = q_s + (size_t)rows_max * width;           // [rows_max][rank]
    float* k_s = acc_s + (size_t)rows_max * rank;            // [tile][width + 1]
    float* p_s = k_s + (size_t)p.tile * kstride;             // [warps][tile]
    float* m_s = p_s + LAT_WARPS * p.tile;                   // [rows_max]
    float* l_s = m_s + rows_max;                             // [rows_max]
    long long* base_s = (long long*)(l_s + rows_max + ((rows_max * (width + rank + 2) + p.tile * (kstride + LAT_WARPS)) & 1));

    pdl_launch();
    pdl_wait();
    const int qb = blockIdx.x, hchunk = blockIdx.y, sp = blockIdx.z;
    const int req = p.qblk[qb * 3 + 0], row0 = p.qblk[qb * 3 + 1], nq = p.qblk[qb * 3 + 2];
    if (nq <= 0) return;
    const int h0 = hchunk * p.hc;
    const int nh = min(p.hc, p.H - h0);
    const int pos_last = p.positions[row0 + nq - 1];
    const int lo_first = first_visible(p.positions[row0], p.window);
    // the first tile that holds a key any row sees (tiles start at multiples of `tile`, as split does)
    const int k_begin = max(sp * p.split, (lo_first / p.tile) * p.tile);
    const int k_end = min((sp + 1) * p.split, pos_last + 1);       // exclusive
    if (k_begin >= k_end) return;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_rows = nq * nh;                                    // row r = (query qi, head h0 + g), r = qi * nh + g
    const TQ* ql = (const TQ*)p.q_lat;
    const TR* qr = (const TR*)p.q_raw;
    const int half = p.rot_dims / 2;
    for (int idx = tid; idx < n_rows * width; idx += LAT_THREADS) {
        const int r = idx / width, d = idx - r * width;
        const int qi = r / nh, g = r - qi * nh;
        const int t = row0 + qi, h = h0 + g;
        float v;
        if (d < rank) {
            v = to_float(ql[(size_t)h * p.ql_head + (size_t)t * p.ql_row + d]);
        } else {
            const int e = d - rank;
            const TR* src = qr + (size_t)t * p.qr_row + (size_t)h * p.qr_head + p.qr_off;
            if (e < p.rot_dims) {
                const int i = e >> 1;
                const float u = to_float(src[2 * i]), w = to_float(src[2 * i + 1]);
                const float c = p.cos_sin[((size_t)t * half + i) * 2], sn = p.cos_sin[((size_t)t * half + i) * 2 + 1];
                v = (e & 1) ? (w * c + u * sn) : (u * c - w * sn);
            } else {
                v = to_float(src[e]);
            }
        }
        q_s[idx] = v;
    }
    for (int idx = tid; idx < n_rows * rank; idx += LAT_THREADS) acc_s[idx] = 0.0f;
    for (int r = tid; r < n_rows; r += LAT_THREADS) { m_s[r] = -INFINITY; l_s[r] = 0.0f; }

    const TC* pool = (const TC*)p.pool;
    const int tile = p.tile;
    float* pw = p_s + warp * tile;

    for (int t0 = k_begin; t0 < k_end; t0 += tile) {               // k_begin is a multiple of split, split of tile
        __syncthreads();
        for (int j = tid; j < tile; j += LAT_THREADS) {
            const int key = t0 + j;
            long long off = -1;
            if (key >= lo_first && key < k_end) {      // (a key in front of every row's window may lie in a page given back)
                const int page = p.block_table[(size_t)req * p.max_pages + key / p.page_size];
                if (page < 0 || page >= p.num_pages) {
                    if (p.status) atomicOr(p.status, BG_STATUS_BAD_PAGE);
                } else {
                    off = (long long)(((size_t)page * p.page_size + key % p.page_size) * width);
                }
            }
            base_s[j] = off;
        }
        __syncthreads();
        // a warp per key row, four loads of a lane on their way at a time (a load that waited for the store of the
        // one before it left the kernel bound by the latency of single loads)
        for (int j = warp; j < tile; j += LAT_WARPS) {
            const long long off = base_s[j];
            float* dst = k_s + j * kstride;
            if (off < 0) {
                for (int d = lane; d < width; d += 32) dst[d] = 0.0f;
                continue;
            }
            const TC* srow = pool + off;
            int d = lane;
            for (; d + 96 < width; d += 128) {
                const TC a0 = srow[d], a1 = srow[d + 32], a2 = srow[d + 64], a3 = srow[d + 96];
                dst[d] = to_float(a0); dst[d + 32] = to_float(a1); dst[d + 64] = to_float(a2); dst[d + 96] = to_float(a3);
            }
            for (; d < width; d += 32) dst[d] = to_float(srow[d]);
        }
        __syncthreads();

        for (int r = warp; r < n_rows; r += LAT_WARPS) {
            const int qi = r / nh;
            const int pos = p.positions[row0 + qi];
            const int lo = first_visible(pos, p.window);
            const float* qrow = q_s + (size_t)r * width;
            float s[2];
            float tmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s[c] = -INFINITY;
                const int j = c * 32 + lane;
                if (j < tile) {
                    const int key = t0 + j;
                    if (key >= lo && key <= pos && key < k_end && base_s[j] >= 0) {
                        const float* kr = k_s + j * kstride;
                        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;      // four chains, joined in a fixed order
                        int d = 0;
                        for (; d + 3 < width; d += 4) {
                            d0 = fmaf(qrow[d], kr[d], d0);
                            d1 = fmaf(qrow[d + 1], kr[d + 1], d1);
                            d2 = fmaf(qrow[d + 2], kr[d + 2], d2);
                            d3 = fmaf(qrow[d + 3], kr[d + 3], d3);
                        }
                        for (; d < width; ++d) d0 = fmaf(qrow[d], kr[d], d0);
                        s[c] = ((d0 + d1) + (d2 + d3)) * p.scale;
                    }
                }
                tmax = fmaxf(tmax, s[c]);
            }
            tmax = warp_max(tmax);
            if (tmax == -INFINITY) continue;                       // no visible key of this tile for this row
            const float m_old = m_s[r];
            const float m_new = fmaxf(m_old, tmax);
            const float corr = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
            float psum = 0.0f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s[c] = (s[c] == -INFINITY) ? 0.0f : expf(s[c] - m_new);
                psum += s[c];
                if (c * 32 + lane < tile) pw[c * 32 + lane] = s[c];
            }
            psum = warp_sum(psum);
            __syncwarp();
            float* ar = acc_s + (size_t)r * rank;
            int d = lane;
            for (; d + 96 < rank; d += 128) {                      // four features of a lane at a time
                float a0 = ar[d] * corr, a1 = ar[d + 32] * corr, a2 = ar[d + 64] * corr, a3 = ar[d + 96] * corr;
                for (int jj = 0; jj < tile; ++jj) {
                    const float pj = pw[jj];
                    const float* kr = k_s + jj * kstride + d;
                    a0 = fmaf(pj, kr[0], a0); a1 = fmaf(pj, kr[32], a1); a2 = fmaf(pj, kr[64], a2); a3 = fmaf(pj, kr[96], a3);
                }
                ar[d] = a0; ar[d + 32] = a1; ar[d + 64] = a2; ar[d + 96] = a3;
            }
            for (; d < rank; d += 32) {
                float a = ar[d] * corr;
                for (int jj = 0; jj < tile; ++jj) a = fmaf(pw[jj], k_s[jj * kstride + d], a);
                ar[d] = a;
            }
            if (lane == 0) { m_s[r] = m_new; l_s[r] = l_s[r] * corr + psum; }
            __syncwarp();
        }
    }
    __syncthreads();
    // partial results, only for rows that see at least one key of this split
    for (int r = warp; r < n_rows; r += LAT_WARPS) {
        const int qi = r / nh, g = r - qi * nh;
        const int pos = p.positions[row0 + qi];
        if (pos < sp * p.split || first_visible(pos, p.window) >= (sp + 1) * p.split) continue;
        const size_t prow = ((size_t)(row0 + qi) * p.H + h0 + g) * p.max_splits + sp;
        for (int d = lane; d < rank; d += 32) p.part_o[prow * rank + d] = acc_s[(size_t)r * rank + d];
        if (lane == 0) { p.part_ml[prow * 2 + 0] = m_s[r]; p.part_ml[prow * 2 + 1] = l_s[r]; }
    }
}

// out[h][t][:] = sum_s o_s e^(m_s - m) / sum_s l_s e^(m_s - m) over the splits that hold a key the row sees, in split
// order.  One block of 128 threads per (row, head): the splits' weights are worked out once, by the first warp, and
// every thread then sums its features over the splits with all its loads independent of one another (a warp per
// (row, head) that recomputed the weights for every 32 features took 32 us for 96 rows of 17 splits).
constexpr int LAT_MERGE_THREADS = 128;
template <typename TO>
__global__ void __launch_bounds__(LAT_MERGE_THREADS)
latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                              const int* __restrict__ positions, TO* __restrict__ out, long long out_head,
                              int out_row, int T, int H, int rank, int max_splits, int split, int window) {
    extern __shared__ float f_s[];                 // [max_splits] weights e^(m_s - m) / l
    pdl_launch();
    pdl_wait();
    const int w = blockIdx.x;
    const int t = w / H, h = w - t * H;
    const int s_hi = positions[t] / split;
    const int s_lo = first_visible(positions[t], window) / split;
    const size_t prow = (size_t)w * max_splits;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x < 32) {
        float m = -INFINITY;
        for (int s = s_lo + lane; s <= s_hi; s += 32) m = fmaxf(m, part_ml[(prow + s) * 2]);
        m = warp_max(m);
        float l = 0.0f;
        for (int s = s_lo; s <= s_hi; ++s) l = fmaf(part_ml[(prow + s) * 2 + 1], expf(part_ml[(prow + s) * 2] - m), l);
        const float inv = 1.0f / l;
        for (int s = s_lo + lane; s <= s_hi; s += 32) f_s[s] = expf(part_ml[(prow + s) * 2] - m) * inv;
    }
    __syncthreads();
    TO* o = out + (size_t)h * out_head + (size_t)t * out_row;
    for (int d = threadIdx.x; d < rank; d += LAT_MERGE_THREADS) {
        float acc = 0.0f;
        for (int s = s_lo; s <= s_hi; ++s) acc = fmaf(part_o[(prow + s) * rank + d], f_s[s], acc);
        o[d] = from_float<TO>(acc);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The other way round, for long prompt portions in bfloat16: make every head's keys and values of the request's
// positions once per step (one product of the cached latents with [W_uk; W_uv]) and hand them, laid out as pages
// of 64 positions of a pool of the step's own, to the grouped-query kernel on the tensor cores.  Per key and
// head that costs dim + vdim features instead of rank + rot, and the products run at matrix speed.  Three
// small kernels: the request's cached rows gathered into a matrix, the per-head rows put into pages (keys with the
// shared rotated part behind them), and the rotation of the queries' rot part in place.

// lat[s, :] and kr[s, :] = the latent and the rotated key part of the cached row of position first + s of request `req`,
// zeros where the block table holds no page.  Two matrices, so that the product that follows reads a dense one.
__global__ void latent_gather_kernel(const __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table, int max_pages,
                                     int req, int num_pages, int page_size, int rank, int rot, int S, int first,
                                     __nv_bfloat16* __restrict__ lat, __nv_bfloat16* __restrict__ kr) {
    pdl_launch();
    pdl_wait();
    const int s = blockIdx.x;
    if (s >= S) return;
    const int width = rank + rot;
    const int at = first + s;                                  // the position whose row this is
    const int page = at / page_size < max_pages ? block_table[(size_t)req * max_pages + at / page_size] : -1;
    const bool ok = page >= 0 && page < num_pages;
    const __nv_bfloat16* src = pool + ((size_t)(ok ? page : 0) * page_size + at % page_size) * width;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
    if ((width & 7) == 0 && (rank & 7) == 0) {                 // rows and both parts on 16-byte boundaries
        for (int c = threadIdx.x; c < width / 8; c += blockDim.x) {
            const uint4 v = ok ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
            __nv_bfloat16* dst = c * 8 < rank ? lat + (size_t)s * rank + c * 8 : kr + (size_t)s * rot + (c * 8 - rank);
            *reinterpret_cast<uint4*>(dst) = v;
        }
        return;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        const __nv_bfloat16 v = ok ? src[d] : zero;
        if (d < rank) lat[(size_t)s * rank + d] = v;
        else kr[(size_t)s * rot + d - rank] = v;
    }
}

// kv[s] = [k_plain (H x dim) | v (H x hd)] and kr[s] = the rotated key part (rot), hd = dim + rot:
// pages[s / 64][0][h][s % 64] = [k_plain_h | key part], pages[s / 64][1][h][s % 64] = v_h.  A thread moves 16 bytes
// (dim and rot are multiples of 8 wherever the grouped-query kernel takes the head size).
__global__ void latent_expand_kernel(const __nv_bfloat16* __restrict__ kv, int kv_stride, const __nv_bfloat16* __restrict__ kr,
                                     int H, int dim, int rot, int S, __nv_bfloat16* __restrict__ pages) {
    pdl_launch();
    pdl_wait();
    const int hd = dim + rot, cpr = hd / 8;                    // 16-byte pieces per row
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = (size_t)S * H * 2 * cpr;
    if (i >= n) return;
    const int c = (int)(i % cpr);
    const int kvsel = (int)((i / cpr) % 2);
    const int h = (int)((i / ((size_t)cpr * 2)) % H);
    const int s = (int)(i / ((size_t)cpr * 2 * H));
    const size_t page_elems = (size_t)2 * H * 64 * hd;
    __nv_bfloat16* dst = pages + (size_t)(s / 64) * page_elems + (size_t)kvsel * H * 64 * hd + ((size_t)h * 64 + s % 64) * hd + c * 8;
    const __nv_bfloat16* src;
    if (kvsel) src = kv + (size_t)s * kv_stride + (size_t)H * dim + (size_t)h * hd + c * 8;
    else if (c * 8 < dim) src = kv + (size_t)s * kv_stride + (size_t)h * dim + c * 8;
    else src = kr + (size_t)s * rot + (c * 8 - dim);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
}

// q[t, h, off + 2i], q[t, h, off + 2i + 1] turn by cos_sin[t, i] for i < rot_dims / 2, in place.
__global__ void rotate_q_kernel(__nv_bfloat16* __restrict__ q, int q_stride, int head, int off, int rot_dims, int H,
                                const float* __restrict__ cos_sin, int T) {
    pdl_launch();
    pdl_wait();
    const int half = rot_dims / 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)T * H * half) return;
    const int k = (int)(i % half);
    const int h = (int)((i / half) % H);
    const int t = (int)(i / ((size_t)half * H));
    __nv_bfloat16* p = q + (size_t)t * q_stride + (size_t)h * head + off + 2 * k;
    const float u = __bfloat162float(p[0]), v = __bfloat162float(p[1]);
    const float c = cos_sin[((size_t)t * half + k) * 2], sn = cos_sin[((size_t)t * half + k) * 2 + 1];
    p[0] = __float2bfloat16_rn(u * c - v * sn);
    p[1] = __float2bfloat16_rn(v * c + u * sn);
}

}  // namespace bg

using namespace bg;

static size_t latent_smem_bytes(int rows, int rank, int rot, int tile) {
    const size_t width = (size_t)rank + rot;
    size_t floats = (size_t)rows * (width + rank + 2) + (size_t)tile * (width + 1 + LAT_WARPS);
    floats += floats & 1;
    return floats * sizeof(float) + (size_t)tile * sizeof(long long);
}

// Rows per CTA (queries x heads) and keys per tile that fit one CTA's shared memory for these sizes.
extern "C" int bg_latent_attention_plan(int rank, int rot, int* rows_out, int* tile_out) {
    if (rank <= 0 || rot < 0) return BG_ERR_UNSUPPORTED;
    const size_t limit = 200 * 1024;
    for (int rows = 64; rows >= 1; rows >>= 1) {
        for (int tile = 64; tile >= 32; tile >>= 1) {
            if (latent_smem_bytes(rows, rank, rot, tile) <= limit) { *rows_out = rows; *tile_out = tile; return BG_OK; }
        }
    }
    return BG_ERR_UNSUPPORTED;
}

extern "C" int bg_latent_append(const void* src, int src_dtype, int src_stride, int col0, int rank, int rot, int rot_dims,
                                const void* w, int w_dtype, float eps, const float* cos_sin, const int* positions,
                                const int* row_req, const int* block_table, int max_pages, void* pool, int pool_dtype,
                                int num_pages, int page_size, int n_rows, unsigned* status, int q_col0, int q_rank,
                                const void* q_w, void* q_out, int q_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return BG_OK;
    if (rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return BG_ERR_SHAPE;
    if (q_out && q_rank <= 0) return BG_ERR_SHAPE;
    if (!q_out) q_dtype = pool_dtype;
    BG_DISPATCH_DTYPE(src_dtype, TI, BG_DISPATCH_DTYPE(w_dtype, TW, BG_DISPATCH_DTYPE(pool_dtype, TC, BG_DISPATCH_DTYPE(q_dtype, TQ,
        launch(latent_append_kernel<TI, TW, TC, TQ>, dim3(n_rows), dim3(128), 0, stream, (const TI*)src, src_stride, col0, rank,
               rot, rot_dims, (const TW*)w, eps, cos_sin, positions, row_req, block_table, max_pages, (TC*)pool, num_pages,
               page_size, status, q_col0, q_rank, (const TW*)q_w, (TQ*)q_out)))));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_latent_attention_partial(const void* q_lat, int ql_dtype, long long ql_head, int ql_row, const void* q_raw,
                                           int qr_dtype, int qr_row, int qr_head, int qr_off, const float* cos_sin,
                                           const void* pool, int pool_dtype, int num_pages, int page_size,
                                           const int* block_table, int max_pages, const int* positions, const int* qblk,
                                           int n_qblk, float* part_o, float* part_ml, int max_splits, int n_splits_launch,
                                           int H, int hc, int rank, int rot, int rot_dims, int split, int tile, int bq,
                                           int window, float scale, unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0 || n_splits_launch <= 0) return BG_OK;
    if (H <= 0 || hc <= 0 || hc > H || rank <= 0 || rot < 0 || rot_dims > rot || (rot_dims & 1)) return BG_ERR_SHAPE;
    if ((tile != 32 && tile != 64) || split % tile != 0 || bq <= 0) return BG_ERR_SHAPE;
    const int chunks = (H + hc - 1) / hc;
    if (n_splits_launch > max_splits || n_splits_launch > 65535 || chunks > 65535) return BG_ERR_SHAPE;
    LatentParams p;
    p.q_lat = q_lat; p.ql_head = ql_head; p.ql_row = ql_row; p.q_raw = q_raw; p.qr_row = qr_row; p.qr_head = qr_head;
    p.qr_off = qr_off; p.cos_sin = cos_sin; p.pool = pool; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.max_pages = max_pages; p.positions = positions; p.qblk = qblk; p.part_o = part_o;
    p.part_ml = part_ml; p.max_splits = max_splits; p.H = H; p.hc = hc; p.rank = rank; p.rot = rot; p.rot_dims = rot_dims;
    p.split = split; p.tile = tile; p.bq = bq; p.window = window; p.scale = scale; p.status = status;
    const size_t smem = latent_smem_bytes(bq * hc, rank, rot, tile);
    if (smem > 227 * 1024) return BG_ERR_UNSUPPORTED;
    dim3 grid(n_qblk, chunks, n_splits_launch);
#define BG_LAT_LAUNCH(TQ, TR, TC)                                                                          \
    do {                                                                                                   \
        auto kern = latent_attention_partial_kernel<TQ, TR, TC>;                                           \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e;                                                               \
        launch(kern, grid, dim3(LAT_THREADS), smem, stream, p);                                            \
    } while (0)
    if (ql_dtype != BG_DTYPE_F32) return BG_ERR_DTYPE;             // the queries in the latent space come as float
    if (qr_dtype == BG_DTYPE_F32 && pool_dtype == BG_DTYPE_F32) BG_LAT_LAUNCH(float, float, float);
    else if (qr_dtype == BG_DTYPE_BF16 && pool_dtype == BG_DTYPE_BF16) BG_LAT_LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
    else if (qr_dtype == BG_DTYPE_F32 && pool_dtype == BG_DTYPE_BF16) BG_LAT_LAUNCH(float, float, __nv_bfloat16);
    else if (qr_dtype == BG_DTYPE_BF16 && pool_dtype == BG_DTYPE_F32) BG_LAT_LAUNCH(float, __nv_bfloat16, float);
    else return BG_ERR_DTYPE;
#undef BG_LAT_LAUNCH
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_latent_attention_merge(const float* part_o, const float* part_ml, const int* positions, void* out,
                                         int out_dtype, long long out_head, int out_row, int T, int H, int rank,
                                         int max_splits, int split, int window, cudaStream_t stream) {
    const long long blocks = (long long)T * H;
    if (blocks <= 0) return BG_OK;
    if (blocks > 0x7fffffffLL || max_splits > 8192) return BG_ERR_SHAPE;
    BG_DISPATCH_DTYPE(out_dtype, TO,
        launch(latent_attention_merge_kernel<TO>, dim3((unsigned)blocks), dim3(LAT_MERGE_THREADS), (size_t)max_splits * sizeof(float),
               stream, part_o, part_ml, positions, (TO*)out, out_head, out_row, T, H, rank, max_splits, split, window));
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_latent_gather(const void* pool, const int* block_table, int max_pages, int req, int num_pages, int page_size,
                                int rank, int rot, int S, int first, void* lat, void* kr, cudaStream_t stream) {
    if (S <= 0) return BG_OK;
    launch(latent_gather_kernel, dim3(S), dim3(64), 0, stream, (const __nv_bfloat16*)pool, block_table, max_pages, req, num_pages,
           page_size, rank, rot, S, first, (__nv_bfloat16*)lat, (__nv_bfloat16*)kr);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_latent_expand(const void* kv, int kv_stride, const void* kr, int H, int dim, int rot, int S, void* pages,
                                cudaStream_t stream) {
    if (S <= 0) return BG_OK;
    if (H <= 0 || dim % 8 != 0 || rot % 8 != 0 || kv_stride % 8 != 0) return BG_ERR_SHAPE;
    const size_t n = (size_t)S * H * 2 * ((dim + rot) / 8);
    launch(latent_expand_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)kv, kv_stride,
           (const __nv_bfloat16*)kr, H, dim, rot, S, (__nv_bfloat16*)pages);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

extern "C" int bg_rotate_q(void* q, int q_stride, int head, int off, int rot_dims, int H, const float* cos_sin, int T,
                           cudaStream_t stream) {
    const long long n = (long long)T * H * (rot_dims / 2);
    if (n <= 0) return BG_OK;
    if (rot_dims & 1) return BG_ERR_SHAPE;
    launch(rotate_q_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (__nv_bfloat16*)q, q_stride, head, off, rot_dims,
           H, cos_sin, T);
    BG_LAUNCH_CHECK();
    return BG_OK;
}
