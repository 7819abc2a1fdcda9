// Attention through a latent on the tensor cores, for steps of single tokens and short portions in bfloat16:
// the same work layout, arguments and partial results as latent_attention.cu (a CTA per (query block, chunk of
// heads, split of the keys); a running maximum, sum and unnormalised result per (row, head); the same merge
// kernel behind it), with the two products of a tile of 64 keys as mma.sync m16n8k16 on bfloat16 operands with
// float accumulation.
//
// All heads of a row score against the SAME cached rows, so the rows of a CTA (queries x heads, up to 64) are the
// M side of both products: S[rows, 64] = Q[rows, width] K[64, width]^T and O[rows, rank] += P[rows, 64] V[64, rank],
// V being the first `rank` features of K.  Eight warps: for the scores a warp takes eight keys of the tile for all
// rows; the softmax runs a warp per row over shared memory (float); for the values a warp owns tiles of eight
// value features for all rows, its accumulators in registers across the tiles of keys.  The key tiles come by
// 16-byte cp.async, the next tile under way while the current one is computed when two tiles fit shared memory.
#include "common.cuh"

namespace bg {

constexpr int LM_THREADS = 256;
constexpr int LM_WARPS = 8;
constexpr int LM_TILE = 64;
constexpr int LM_SS = LM_TILE + 1;       // floats per row of scores
constexpr int LM_PS = LM_TILE + 8;       // bf16 per row of weights

struct LatentMmaParams {
    const float* q_lat;     // [H][T][rank] float
    long long ql_head;
    int ql_row;
    const __nv_bfloat16* q_raw;   // [T][H][dim + rot]
    int qr_row, qr_head, qr_off;
    const float* cos_sin;
    const __nv_bfloat16* pool;    // [num_pages][page_size][rank + rot]
    int num_pages, page_size;
    const int* block_table;
    int max_pages;
    const int* positions;
    const int* qblk;
    float* part_o;
    float* part_ml;
    int max_splits;
    int H, hc;
    int rank, rot, rot_dims;
    int split, bq, stages;
    int window;             // as first_visible() reads it; 0: every earlier position
    float scale;
    unsigned* status;
};

__device__ __forceinline__ void lm_cp_async16(void* smem_dst, const void* gmem_src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void lm_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void lm_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void lm_ldmatrix_x4(unsigned (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MT: tiles of 16 rows; NT: tiles of 8 value features per warp (warp w owns feature tiles w, w + 8, ...).
template <int MT, int NT>
__global__ void __launch_bounds__(LM_THREADS)
latent_attention_mma_kernel(LatentMmaParams p) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int rank = p.rank, width = p.rank + p.rot;
    const int ks_stride = width + 8;                         // bf16 per row of Q and K in shared memory
    constexpr int ROWS = MT * 16;
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);                       // [ROWS][ks_stride]
    __nv_bfloat16* k_s = q_s + (size_t)ROWS * ks_stride;                                  // [stages][64][ks_stride]
    __nv_bfloat16* p_s = k_s + (size_t)p.stages * LM_TILE * ks_stride;                    // [ROWS][LM_PS]
    float* s_s = reinterpret_cast<float*>(p_s + ROWS * LM_PS);                            // [ROWS][LM_SS]
    float* m_s = s_s + ROWS * LM_SS;                                                      // [ROWS]
    float* l_s = m_s + ROWS;
    float* corr_s = l_s + ROWS;
    int* pos_s = reinterpret_cast<int*>(corr_s + ROWS);                                   // [ROWS] position, -1: no row
    int* lo_s = pos_s + ROWS;                                                             // [ROWS] the first key the row sees
    int* ok_s = lo_s + ROWS;                                                              // [stages][64] the key has a page

    pdl_launch();
    pdl_wait();
    const int qb = blockIdx.x, hchunk = blockIdx.y, sp = blockIdx.z;
    const int req = p.qblk[qb * 3 + 0], row0 = p.qblk[qb * 3 + 1], nq = p.qblk[qb * 3 + 2];
    if (nq <= 0) return;
    const int h0 = hchunk * p.hc;
    const int nh = min(p.hc, p.H - h0);
    const int pos_last = p.positions[row0 + nq - 1];
    const int lo_first = first_visible(p.positions[row0], p.window);
    // the first tile that holds a key any row sees (tiles start at multiples of LM_TILE, as split does)
    const int k_begin = max(sp * p.split, (lo_first / LM_TILE) * LM_TILE);
    const int k_end = min((sp + 1) * p.split, pos_last + 1);
    if (k_begin >= k_end) return;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int n_rows = nq * nh;                                    // row r = (query r / nh, head h0 + r % nh)
    const int half = p.rot_dims / 2;
    // the rows' queries as bfloat16: a warp per row, the latent part with four loads of a lane on their way at a time
    for (int r = warp; r < ROWS; r += LM_WARPS) {
        __nv_bfloat16* qd = q_s + (size_t)r * ks_stride;
        if (r >= n_rows) {
            for (int d = lane; d < width; d += 32) qd[d] = __float2bfloat16_rn(0.0f);
            continue;
        }
        const int qi = r / nh, hh = r - qi * nh;
        const int t = row0 + qi, h = h0 + hh;
        const float* ql = p.q_lat + (size_t)h * p.ql_head + (size_t)t * p.ql_row;
        int d = lane;
        for (; d + 96 < rank; d += 128) {
            const float a0 = ql[d], a1 = ql[d + 32], a2 = ql[d + 64], a3 = ql[d + 96];
            qd[d] = __float2bfloat16_rn(a0); qd[d + 32] = __float2bfloat16_rn(a1);
            qd[d + 64] = __float2bfloat16_rn(a2); qd[d + 96] = __float2bfloat16_rn(a3);
        }
        for (; d < rank; d += 32) qd[d] = __float2bfloat16_rn(ql[d]);
        const __nv_bfloat16* src = p.q_raw + (size_t)t * p.qr_row + (size_t)h * p.qr_head + p.qr_off;
        for (int i = lane; i < half; i += 32) {
            const float u = __bfloat162float(src[2 * i]), w = __bfloat162float(src[2 * i + 1]);
            const float c = p.cos_sin[((size_t)t * half + i) * 2], sn = p.cos_sin[((size_t)t * half + i) * 2 + 1];
            qd[rank + 2 * i] = __float2bfloat16_rn(u * c - w * sn);
            qd[rank + 2 * i + 1] = __float2bfloat16_rn(w * c + u * sn);
        }
        for (int e = p.rot_dims + lane; e < p.rot; e += 32) qd[rank + e] = src[e];
    }
    for (int r = tid; r < ROWS; r += LM_THREADS) {
        m_s[r] = -INFINITY; l_s[r] = 0.0f; corr_s[r] = 1.0f;
        pos_s[r] = r < n_rows ? p.positions[row0 + r / nh] : -1;
        lo_s[r] = r < n_rows ? first_visible(pos_s[r], p.window) : 0;
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][j][e] = 0.0f;

    const int chunks = width / 8;                                  // 16-byte pieces of a cached row
    const int n_tiles = (k_end - k_begin + LM_TILE - 1) / LM_TILE;
    const int n_ftiles = rank / 8;

    // brings tile `ti` into stage `st`: every key's row by cp.async, zeros for keys beyond the split or without a page
    auto fetch = [&](int ti, int st) {
        const int t0 = k_begin + ti * LM_TILE;
        __nv_bfloat16* kd = k_s + (size_t)st * LM_TILE * ks_stride;
        const int j = tid >> 2, c0 = tid & 3;                      // four threads share a key's row
        const int key = t0 + j;
        bool ok = false;
        const __nv_bfloat16* src = nullptr;
        if (key >= lo_first && key < k_end) {          // (a key in front of every row's window may lie in a page given back)
            const int page = p.block_table[(size_t)req * p.max_pages + key / p.page_size];
            if (page < 0 || page >= p.num_pages) {
                if (p.status && c0 == 0) atomicOr(p.status, BG_STATUS_BAD_PAGE);
            } else {
                ok = true;
                src = p.pool + ((size_t)page * p.page_size + key % p.page_size) * width;
            }
        }
        __nv_bfloat16* dst = kd + (size_t)j * ks_stride;
        if (ok) {
            for (int c = c0; c < chunks; c += 4) lm_cp_async16(dst + c * 8, src + c * 8);
        } else {
            for (int c = c0; c < chunks; c += 4) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (c0 == 0) ok_s[st * LM_TILE + j] = ok ? 1 : 0;
        lm_cp_async_commit();
    };

    fetch(0, 0);
    for (int ti = 0; ti < n_tiles; ++ti) {
        const int st = p.stages == 2 ? (ti & 1) : 0;
        if (p.stages == 2 && ti + 1 < n_tiles) {
            fetch(ti + 1, (ti + 1) & 1);
            lm_cp_async_wait<1>();
        } else {
            lm_cp_async_wait<0>();
        }
        __syncthreads();
        const int t0 = k_begin + ti * LM_TILE;
        const __nv_bfloat16* kt = k_s + (size_t)st * LM_TILE * ks_stride;
        const int* okt = ok_s + st * LM_TILE;

        // ---- scores: this warp's eight keys (8 warp .. 8 warp + 7) against all rows
        {
            float sc[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[mt][e] = 0.0f;
            const __nv_bfloat16* kb = kt + (size_t)(warp * 8 + (lane & 7)) * ks_stride + (lane >> 3) * 8;
            const __nv_bfloat16* qa = q_s + (size_t)(lane & 15) * ks_stride + (lane >> 4) * 8;
            for (int f0 = 0; f0 < width; f0 += 32) {               // two steps of 16 features per B load
                unsigned b[4];
                lm_ldmatrix_x4(b, kb + f0);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    unsigned a[4];
                    lm_ldmatrix_x4(a, qa + (size_t)mt * 16 * ks_stride + f0);
                    lm_mma(sc[mt], a, b[0], b[1]);
                    lm_ldmatrix_x4(a, qa + (size_t)mt * 16 * ks_stride + f0 + 16);
                    lm_mma(sc[mt], a, b[2], b[3]);
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = mt * 16 + g + (e >> 1) * 8;
                    const int j = warp * 8 + 2 * t4 + (e & 1);
                    const int key = t0 + j;
                    const bool seen = key >= lo_s[r] && key <= pos_s[r] && key < k_end && okt[j];
                    s_s[r * LM_SS + j] = seen ? sc[mt][e] * p.scale : -INFINITY;
                }
        }
        __syncthreads();

        // ---- softmax: a warp per row
        for (int r = warp; r < ROWS; r += LM_WARPS) {
            const float s0 = s_s[r * LM_SS + lane], s1 = s_s[r * LM_SS + 32 + lane];
            const float tmax = warp_max(fmaxf(s0, s1));
            __nv_bfloat16* pr = p_s + r * LM_PS;
            if (tmax == -INFINITY) {                               // the row sees no key of this tile
                pr[lane] = __float2bfloat16_rn(0.0f);
                pr[32 + lane] = __float2bfloat16_rn(0.0f);
                if (lane == 0) corr_s[r] = 1.0f;
                continue;
            }
            const float m_old = m_s[r];
            const float m_new = fmaxf(m_old, tmax);
            const float corr = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
            const float p0 = (s0 == -INFINITY) ? 0.0f : expf(s0 - m_new);
            const float p1 = (s1 == -INFINITY) ? 0.0f : expf(s1 - m_new);
            const float psum = warp_sum(p0 + p1);
            pr[lane] = __float2bfloat16_rn(p0);
            pr[32 + lane] = __float2bfloat16_rn(p1);
            if (lane == 0) { m_s[r] = m_new; l_s[r] = l_s[r] * corr + psum; corr_s[r] = corr; }
        }
        __syncthreads();

        // ---- values: this warp's feature tiles for all rows
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const float c_lo = corr_s[mt * 16 + g], c_hi = corr_s[mt * 16 + g + 8];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                acc[mt][j][0] *= c_lo; acc[mt][j][1] *= c_lo; acc[mt][j][2] *= c_hi; acc[mt][j][3] *= c_hi;
            }
        }
        const __nv_bfloat16* pa = p_s + (lane & 15) * LM_PS + (lane >> 4) * 8;
#pragma unroll
        for (int kk = 0; kk < LM_TILE / 16; ++kk) {
            unsigned a[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) lm_ldmatrix_x4(a[mt], pa + mt * 16 * LM_PS + kk * 16);
            const __nv_bfloat16* vrow = kt + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ks_stride;
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                const int f_a = warp + 8 * j, f_b = warp + 8 * (j + 1);
                const bool has_a = f_a < n_ftiles, has_b = (j + 1 < NT) && f_b < n_ftiles;
                if (!has_a) break;                                 // uniform over the warp
                unsigned b[4];
                lm_ldmatrix_x4_trans(b, vrow + ((lane >> 4) && has_b ? f_b : f_a) * 8);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    lm_mma(acc[mt][j], a[mt], b[0], b[1]);
                    if (j + 1 < NT) {
                        if (has_b) lm_mma(acc[mt][j + 1 < NT ? j + 1 : j], a[mt], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                                           // the stage and the weights may be overwritten
    }

    // ---- partial results of the rows that see a key of this split
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int r = mt * 16 + g + hi * 8;
            if (r >= n_rows || pos_s[r] < sp * p.split || lo_s[r] >= (sp + 1) * p.split) continue;
            const int qi = r / nh, hh = r - qi * nh;
            const size_t prow = ((size_t)(row0 + qi) * p.H + h0 + hh) * p.max_splits + sp;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int f = warp + 8 * j;
                if (f < n_ftiles) {
                    float2 v = make_float2(acc[mt][j][hi * 2], acc[mt][j][hi * 2 + 1]);
                    *reinterpret_cast<float2*>(p.part_o + prow * rank + f * 8 + 2 * t4) = v;
                }
            }
        }
    for (int r = tid; r < n_rows; r += LM_THREADS) {
        if (pos_s[r] < sp * p.split || lo_s[r] >= (sp + 1) * p.split) continue;
        const int qi = r / nh, hh = r - qi * nh;
        const size_t prow = ((size_t)(row0 + qi) * p.H + h0 + hh) * p.max_splits + sp;
        p.part_ml[prow * 2 + 0] = m_s[r];
        p.part_ml[prow * 2 + 1] = l_s[r];
    }
}

}  // namespace bg

using namespace bg;

static size_t latent_mma_smem(int rows, int width, int stages) {
    const size_t ks = (size_t)width + 8;
    size_t b = (size_t)rows * ks * 2 + (size_t)stages * LM_TILE * ks * 2 + (size_t)rows * LM_PS * 2 + (size_t)rows * LM_SS * 4 +
               (size_t)rows * 5 * 4 + (size_t)stages * LM_TILE * 4;
    return (b + 15) / 16 * 16;
}

// Whether the tensor-core kernel takes these sizes, and with how many rows per CTA (16, 32 or 64) and stages (1 or 2).
extern "C" int bg_latent_attention_mma_plan(int rank, int rot, int* rows_out, int* stages_out) {
    const int width = rank + rot;
    if (rank <= 0 || rot < 0 || width % 32 != 0 || rank % 8 != 0 || rank > 512) return BG_ERR_UNSUPPORTED;
    const size_t limit = 200 * 1024;
    for (int rows = 64; rows >= 16; rows >>= 1) {
        if (rows == 64 && rank > 256) continue;                    // 64 rows x 512 features would not fit the registers
        for (int stages = 2; stages >= 1; --stages)
            if (latent_mma_smem(rows, width, stages) <= limit) { *rows_out = rows; *stages_out = stages; return BG_OK; }
    }
    return BG_ERR_UNSUPPORTED;
}

extern "C" int bg_latent_attention_mma_partial(const float* q_lat, long long ql_head, int ql_row, const void* q_raw, int qr_row,
                                               int qr_head, int qr_off, const float* cos_sin, const void* pool, int num_pages,
                                               int page_size, const int* block_table, int max_pages, const int* positions,
                                               const int* qblk, int n_qblk, float* part_o, float* part_ml, int max_splits,
                                               int n_splits_launch, int H, int hc, int rank, int rot, int rot_dims, int split,
                                               int bq, int stages, int window, float scale, unsigned* status, cudaStream_t stream) {
    if (n_qblk <= 0 || n_splits_launch <= 0) return BG_OK;
    const int width = rank + rot;
    if (H <= 0 || hc <= 0 || hc > H || width % 32 != 0 || rank % 8 != 0 || rank > 512 || rot_dims > rot || (rot_dims & 1))
        return BG_ERR_SHAPE;
    if (split % LM_TILE != 0 || bq <= 0 || bq * hc > 64) return BG_ERR_SHAPE;
    const int chunks = (H + hc - 1) / hc;
    if (n_splits_launch > max_splits || n_splits_launch > 65535 || chunks > 65535) return BG_ERR_SHAPE;
    const int rows = bq * hc <= 16 ? 16 : (bq * hc <= 32 ? 32 : 64);
    if (rows == 64 && rank > 256) return BG_ERR_UNSUPPORTED;
    LatentMmaParams p;
    p.q_lat = q_lat; p.ql_head = ql_head; p.ql_row = ql_row; p.q_raw = (const __nv_bfloat16*)q_raw; p.qr_row = qr_row;
    p.qr_head = qr_head; p.qr_off = qr_off; p.cos_sin = cos_sin; p.pool = (const __nv_bfloat16*)pool; p.num_pages = num_pages;
    p.page_size = page_size; p.block_table = block_table; p.max_pages = max_pages; p.positions = positions; p.qblk = qblk;
    p.part_o = part_o; p.part_ml = part_ml; p.max_splits = max_splits; p.H = H; p.hc = hc; p.rank = rank; p.rot = rot;
    p.rot_dims = rot_dims; p.split = split; p.bq = bq; p.stages = stages; p.window = window; p.scale = scale; p.status = status;
    // stages: two CTAs on an SM overlap one another's loads, queries and epilogues, so a CTA takes no more than half
    // of an SM's shared memory where it can (with two tiles in flight if they fit that, else with one); a CTA too
    // large for that is alone on its SM and takes two tiles if they fit
    (void)stages;
    const size_t half_sm = 110 * 1024, whole_sm = 200 * 1024;
    const size_t s1 = latent_mma_smem(rows, width, 1), s2 = latent_mma_smem(rows, width, 2);
    stages = s2 <= half_sm ? 2 : (s1 <= half_sm ? 1 : (s2 <= whole_sm ? 2 : 1));
    p.stages = stages;
    const size_t smem = latent_mma_smem(rows, width, stages);
    if (smem > 227 * 1024) return BG_ERR_UNSUPPORTED;
    dim3 grid(n_qblk, chunks, n_splits_launch);
    const int nt = (rank / 8 + LM_WARPS - 1) / LM_WARPS;           // feature tiles per warp: 1 .. 8
#define BG_LM_LAUNCH(MT, NT)                                                                               \
    do {                                                                                                   \
        auto kern = latent_attention_mma_kernel<MT, NT>;                                                   \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e;                                                               \
        launch(kern, grid, dim3(LM_THREADS), smem, stream, p);                                             \
    } while (0)
#define BG_LM_ROWS(MT)                                 \
    do {                                               \
        if (nt <= 1) BG_LM_LAUNCH(MT, 1);              \
        else if (nt <= 2) BG_LM_LAUNCH(MT, 2);         \
        else if (nt <= 4) BG_LM_LAUNCH(MT, 4);         \
        else BG_LM_LAUNCH(MT, 8);                      \
    } while (0)
    if (rows == 16) BG_LM_ROWS(1);
    else if (rows == 32) BG_LM_ROWS(2);
    else {
        if (nt <= 1) BG_LM_LAUNCH(4, 1);
        else if (nt <= 2) BG_LM_LAUNCH(4, 2);
        else BG_LM_LAUNCH(4, 4);
    }
#undef BG_LM_ROWS
#undef BG_LM_LAUNCH
    BG_LAUNCH_CHECK();
    return BG_OK;
}
