// Softmax attention over the paged cache with a sliding window behind which whole blocks of tokens stay in sight as one
// pooled key and value each, a sink per head in the softmax's denominator, a query multiplier that grows with the
// position, and values that may be the keys themselves.  Every one of these is optional, so the same kernels serve plain
// causal attention whose values are its keys and windowed attention with pooled blocks.
//
// Row i of a sequence sees token j if 0 <= i - j < window (window 0: every j <= i), and pooled block b (positions
// b P .. b P + P - 1) if b P + P - 1 <= i - window: the first floor(max(0, i - window + 1) / P) blocks.  Tokens and blocks
// share one softmax; with a sink s_h the denominator also holds exp(s_h).  Head h's scores are (q . k) * scale * m(i) with
// m(i) = 1 + coef * ln(floor((i + 1) / every) + 1), the multiplier applied to the 32-bit score, not to the stored query.
//
//   prepare   per row: q and k heads are RMS-normed with a weight shared by the heads (optional), the first `rot` numbers
//             of each head turn by position (pairs (i, i + rot / 2), angle fp32(pos) * freq[i], cosine and sine times a
//             multiplier; optional); q goes back in place, k and v go to the cache rows of (sequence, position).
//   pool      the block sums: pooled row b of a sequence holds the SUM of the block's keys (and values) as the cache keeps
//             them, in 32-bit, added token by token in the order of positions whatever the steps were (a block that a step
//             continues starts from what the steps before left); readers multiply by 1 / P.  Pooled rows are paged like
//             tokens, 64 to a page.
//   rows      CUDA cores, fp32: a warp per (row, head, split of the keys) with an online softmax, pooled blocks first, then
//             the window; `merge` joins the splits and adds the sink.  One-token steps, and everything in float32.
//   prompt    bf16 prompts on the tensor cores (mma.sync.m16n8k16, fp32 sums): a CTA owns 64 rows of a sequence and one
//             head and walks tiles of 64 pooled rows, then pages of 64 tokens; softmax in fp32; the weights enter the second
//             product as two bf16 numbers each (head and remainder), which keeps them 32-bit in effect.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* attention_pooled_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int PAGE_ROWS = 64;

__device__ __forceinline__ float query_multiplier(int pos, float coef, int every) {
    return every > 0 ? 1.0f + coef * logf((float)((pos + 1) / every) + 1.0f) : 1.0f;
}
__device__ __forceinline__ int blocks_in_sight(int pos, int window, int pool) {
    return (pool > 0 && window > 0) ? max(0, pos - window + 1) / pool : 0;
}

// ------------------------------------------------------------------ prepare
struct PrepArgs {
    void* proj;              // [rows][ld]
    FrVec q_norm, k_norm;    // [dim]; p null: no norm
    const float* freq;       // [rot / 2]; null: no rotation
    void* k_pool;
    void* v_pool;            // null: the values are the keys
    const int* block_table;
    const int* row_seq;
    const int* row_pos;
    int ld, q_off, k_off, v_off, heads, kv_heads, dim, vdim, rot, table_width, rows, write;
    float eps, rot_mult;
};

template <typename T>
__global__ void __launch_bounds__(128) prepare_kernel(PrepArgs p) {
    __shared__ float head_buf[4][256];
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_row = p.heads + 2 * p.kv_heads;              // q heads, k heads, v heads
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)p.rows * per_row) return;
    const int row = (int)(item / per_row), which = (int)(item - (long long)row * per_row);
    const int seq = p.row_seq[row];
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    T* x = (T*)p.proj + (size_t)row * p.ld;
    size_t at = 0;
    if (which >= p.heads) {
        if (!p.write) return;
        const int page = p.block_table[(size_t)seq * p.table_width + pos / PAGE_ROWS];
        at = (size_t)page * PAGE_ROWS + pos % PAGE_ROWS;
    }
    if (which >= p.heads + p.kv_heads) {                        // a value head: copied as it is
        if (p.v_pool == nullptr) return;
        const int g = which - p.heads - p.kv_heads;
        const T* src = x + p.v_off + g * p.vdim;
        T* dst = (T*)p.v_pool + (at * p.kv_heads + g) * p.vdim;
        for (int i = lane; i < p.vdim; i += 32) dst[i] = src[i];
        return;
    }
    const bool is_q = which < p.heads;
    T* src = is_q ? x + p.q_off + which * p.dim : x + p.k_off + (which - p.heads) * p.dim;
    T* dst = is_q ? src : (T*)p.k_pool + (at * p.kv_heads + (which - p.heads)) * p.dim;
    const FrVec& nw = is_q ? p.q_norm : p.k_norm;
    if (nw.p == nullptr && p.freq == nullptr) {
        if (!is_q)
            for (int i = lane; i < p.dim; i += 32) dst[i] = src[i];
        return;
    }
    float* buf = head_buf[warp];
    float ss = 0.f;
    for (int i = lane; i < p.dim; i += 32) {
        const float v = fr_load(src + i);
        buf[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (nw.p != nullptr) {
        const float inv = 1.0f / sqrtf(fr_warp_sum(ss) / (float)p.dim + p.eps);
        for (int i = lane; i < p.dim; i += 32) buf[i] = buf[i] * inv * nw.at(i);
    }
    __syncwarp();
    const int half = p.freq != nullptr ? p.rot / 2 : 0;
    for (int i = lane; i < half; i += 32) {
        float s, c;
        sincosf((float)pos * p.freq[i], &s, &c);
        s *= p.rot_mult;
        c *= p.rot_mult;
        float a, b;
        fr_rotate(buf[i], buf[i + half], c, s, a, b);
        fr_store(dst + i, a);
        fr_store(dst + i + half, b);
    }
    for (int i = 2 * half + lane; i < p.dim; i += 32) fr_store(dst + i, buf[i]);
}

// ------------------------------------------------------------------ pool
struct PoolArgs {
    const void* k_pool;
    const void* v_pool;
    float* pk_pool;          // [pages][64][kv_heads][dim] sums
    float* pv_pool;          // [pages][64][kv_heads][vdim] sums
    const int* block_table;
    const int* pool_table;
    const int* seq_qlen;
    const int* seq_pos0;
    int table_width, pool_table_width, kv_heads, dim, vdim, pool;
};

template <typename T>
__global__ void __launch_bounds__(128) pool_kernel(PoolArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int seq = blockIdx.x, qlen = p.seq_qlen[seq], pos0 = p.seq_pos0[seq];
    if (qlen <= 0) return;
    const int b = pos0 / p.pool + blockIdx.y, last = pos0 + qlen - 1;
    const int j0 = max(b * p.pool, pos0), j1 = min(b * p.pool + p.pool - 1, last);
    if (j0 > j1) return;
    const bool fresh = b * p.pool >= pos0;                      // the block's first token is in this step
    const size_t prow = (size_t)p.pool_table[(size_t)seq * p.pool_table_width + b / PAGE_ROWS] * PAGE_ROWS + b % PAGE_ROWS;
    const int* table = p.block_table + (size_t)seq * p.table_width;
    const int kc = p.kv_heads * p.dim, vc = p.kv_heads * p.vdim;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;       // a thread per channel of the keys, then of the values
    if (c >= kc + vc) return;
    const bool key = c < kc;
    float* dst = key ? p.pk_pool + prow * kc + c : p.pv_pool + prow * vc + (c - kc);
    const T* src = key ? (const T*)p.k_pool + c : (const T*)p.v_pool + (c - kc);
    const int width = key ? kc : vc;
    float acc = fresh ? 0.f : *dst;
    // in the order of positions, four loads in flight
    for (int j = j0; j <= j1; j += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int ju = min(j + u, j1);
            v[u] = fr_load(src + ((size_t)table[ju / PAGE_ROWS] * PAGE_ROWS + ju % PAGE_ROWS) * width);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (j + u <= j1) acc += v[u];
    }
    *dst = acc;
}

// ------------------------------------------------------------------ rows (CUDA cores)
constexpr int MAX_PER_LANE = 8;   // head sizes up to 256

struct RowArgs {
    const void* q;           // [rows][q_stride], head h at q_off + h * dim
    void* out;               // [rows][heads * vdim]
    const void* k_pool;
    const void* v_pool;
    const float* pk_pool;
    const float* pv_pool;
    const int* block_table;
    const int* pool_table;
    const int* row_seq;
    const int* row_pos;
    FrVec sink;              // [heads]; p null: none
    float* part;             // [rows][heads][splits][vdim + 2]
    int table_width, pool_table_width, rows, heads, kv_heads, dim, vdim, q_stride, q_off, window, pool, splits, temp_every;
    float scale, temp_coef;
};

// `count` keys from index `first` of one source: their rows are at row_of(i); four at a time, loads issued together
template <typename KT, typename RowOf>
__device__ __forceinline__ void walk(const RowArgs& p, const KT* kbase, const KT* vbase, int kvh, float kmul, int first, int end, RowOf row_of,
                                     const float (&qv)[MAX_PER_LANE], float (&acc)[MAX_PER_LANE], float& m, float& l, int lane) {
    for (int i = first; i < end; i += 4) {
        const KT* kr[4];
        const KT* vr[4];
        float s4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const size_t at = row_of(min(i + u, end - 1)) * p.kv_heads + kvh;
            kr[u] = kbase + at * p.dim;
            vr[u] = vbase + at * p.vdim;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < MAX_PER_LANE; ++c) {
                const int d = lane + 32 * c;
                if (d < p.dim) s = fmaf(qv[c], fr_load(kr[u] + d), s);
            }
            s4[u] = s;
        }
        float vv[4][MAX_PER_LANE];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int c = 0; c < MAX_PER_LANE; ++c) {
                const int d = lane + 32 * c;
                vv[u][c] = d < p.vdim ? fr_load(vr[u] + d) * kmul : 0.f;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < 4; ++u) s4[u] += __shfl_xor_sync(0xffffffffu, s4[u], o);
        float m_new = m;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            s4[u] *= kmul;
            if (i + u < end) m_new = fmaxf(m_new, s4[u]);
        }
        const float alpha = expf(m - m_new);
        float e4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e4[u] = i + u < end ? expf(s4[u] - m_new) : 0.f;
        l = l * alpha + ((e4[0] + e4[1]) + (e4[2] + e4[3]));
#pragma unroll
        for (int c = 0; c < MAX_PER_LANE; ++c)
            acc[c] = acc[c] * alpha + ((e4[0] * vv[0][c] + e4[1] * vv[1][c]) + (e4[2] * vv[2][c] + e4[3] * vv[3][c]));
        m = m_new;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) rows_kernel(RowArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= p.rows * p.heads) return;
    const int row = item / p.heads, h = item - row * p.heads, split = blockIdx.y;
    const int seq = p.row_seq[row];
    float* part = p.part + ((size_t)item * p.splits + split) * (p.vdim + 2);
    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (seq >= 0) {
        const int pos = p.row_pos[row], kvh = h / (p.heads / p.kv_heads);
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const int n_blocks = blocks_in_sight(pos, p.window, p.pool);
        const int n = n_blocks + pos - lo + 1;
        const int chunk = (n + p.splits - 1) / p.splits;
        const int i0 = split * chunk, i1 = min(i0 + chunk, n);
        const float mult = p.scale * query_multiplier(pos, p.temp_coef, p.temp_every);
        const T* q = (const T*)p.q + (size_t)row * p.q_stride + p.q_off + (size_t)h * p.dim;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            qv[i] = d < p.dim ? fr_load(q + d) * mult : 0.f;
        }
        if (i0 < n_blocks) {
            const int* ptable = p.pool_table + (size_t)seq * p.pool_table_width;
            walk<float>(p, p.pk_pool, p.pv_pool, kvh, 1.0f / (float)p.pool, i0, min(i1, n_blocks),
                        [&](int b) { return (size_t)ptable[b / PAGE_ROWS] * PAGE_ROWS + b % PAGE_ROWS; }, qv, acc, m, l, lane);
        }
        if (i1 > n_blocks) {
            const int* table = p.block_table + (size_t)seq * p.table_width;
            walk<T>(p, (const T*)p.k_pool, (const T*)p.v_pool, kvh, 1.0f, max(i0, n_blocks), i1,
                    [&](int i) { const int j = lo + (i - n_blocks); return (size_t)table[j / PAGE_ROWS] * PAGE_ROWS + j % PAGE_ROWS; }, qv, acc, m, l, lane);
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < p.vdim) part[d] = acc[i];
    }
    if (lane == 0) {
        part[p.vdim] = m;
        part[p.vdim + 1] = l;
    }
}

// o = sum_s o_s exp(m_s - M) / (sum_s l_s exp(m_s - M) + exp(sink - M)), M the largest of the m_s and the sink
template <typename T>
__global__ void __launch_bounds__(128) rows_merge_kernel(RowArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= p.rows * p.heads) return;
    const int h = item % p.heads;
    const float* part = p.part + (size_t)item * p.splits * (p.vdim + 2);
    const bool with_sink = p.sink.p != nullptr && p.row_seq[item / p.heads] >= 0;
    const float sink = with_sink ? p.sink.at(h) : -INFINITY;
    float big = sink;
    for (int s = 0; s < p.splits; ++s) big = fmaxf(big, part[(size_t)s * (p.vdim + 2) + p.vdim]);
    float l = with_sink ? expf(sink - big) : 0.f, acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float* ps = part + (size_t)s * (p.vdim + 2);
        const float ls = ps[p.vdim + 1];
        if (!(ls > 0.f)) continue;
        const float f = expf(ps[p.vdim] - big);
        l += ls * f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < p.vdim) acc[i] += ps[d] * f;
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o_row = (T*)p.out + (size_t)item * p.vdim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < p.vdim) fr_store(o_row + d, acc[i] * inv);
    }
}

// ------------------------------------------------------------------ prompt (tensor cores, bf16)
constexpr int BM = 64, BN = 64, PAD = 8;

struct PromptArgs {
    const bf16* q;           // [rows][q_stride], head h at q_off + h * dim
    bf16* out;               // [rows][heads * vdim]
    const bf16* k_pool;
    const bf16* v_pool;
    const float* pk_pool;
    const float* pv_pool;
    const int* block_table;
    const int* pool_table;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_pos0;
    FrVec sink;
    int table_width, pool_table_width, q_stride, q_off, heads, kv_heads, dim, vdim, window, pool, temp_every;
    float scale, temp_coef;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *(const uint32_t*)&v;
}
// head and remainder of two fp32 weights as packed bf16 pairs
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const bf16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
    const __nv_bfloat162 h = __halves2bfloat162(hx, hy);
    hi = *(const uint32_t*)&h;
    lo = pack2(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

// eight channels from c of a row of `n` channels: bf16 as stored, or 32-bit sums times `mul` rounded to bf16
__device__ __forceinline__ uint4 piece_bf16(const bf16* src, int c, int n) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (c + 8 <= n && (((uintptr_t)(src + c)) & 15) == 0) return *(const uint4*)(src + c);
    bf16* e = (bf16*)&v;
    for (int i = 0; i < 8; ++i) e[i] = c + i < n ? src[c + i] : __float2bfloat16_rn(0.f);
    return v;
}
__device__ __forceinline__ uint4 piece_sum(const float* src, int c, int n, float mul) {
    uint4 v;
    bf16* e = (bf16*)&v;
    for (int i = 0; i < 8; ++i) e[i] = __float2bfloat16_rn(c + i < n ? src[c + i] * mul : 0.f);
    return v;
}

template <int DK, int DV>
__global__ void __launch_bounds__(128, 3) prompt_kernel(PromptArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                           // [BM][DK + PAD]
    bf16* sk = sq + BM * (DK + PAD);                      // [BN][DK + PAD]
    bf16* svt = sk + BN * (DK + PAD);                     // [DV][BN + PAD]
    // the last row tiles first: without a window they walk the most keys, and the short ones then fill the grid's tail
    const int seq = blockIdx.z, h = blockIdx.y, q0 = (gridDim.x - 1 - blockIdx.x) * BM;
    const int qlen = p.seq_qlen[seq];
    if (q0 >= qlen) return;
    const int row0 = p.seq_start[seq] + q0, pos0 = p.seq_pos0[seq] + q0;
    const int n_rows = min(BM, qlen - q0);
    const int kvh = h / (p.heads / p.kv_heads);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    fr_pdl_wait();
    fr_pdl_launch();

    for (int idx = tid; idx < BM * (DK / 8); idx += 128) {
        const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) v = piece_bf16(p.q + (size_t)(row0 + r) * p.q_stride + p.q_off + (size_t)h * p.dim, c, p.dim);
        *(uint4*)(sq + r * (DK + PAD) + c) = v;
    }
    __syncthreads();
    uint32_t qa[DK / 16][4];
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
        const bf16* base = sq + (warp * 16 + g) * (DK + PAD) + ks * 16 + 2 * t;
        qa[ks][0] = *(const uint32_t*)base;
        qa[ks][1] = *(const uint32_t*)(base + 8 * (DK + PAD));
        qa[ks][2] = *(const uint32_t*)(base + 8);
        qa[ks][3] = *(const uint32_t*)(base + 8 * (DK + PAD) + 8);
    }
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int my_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};
    const int last_pos = pos0 + n_rows - 1;
    const float mult[2] = {p.scale * query_multiplier(my_pos[0], p.temp_coef, p.temp_every),
                           p.scale * query_multiplier(my_pos[1], p.temp_coef, p.temp_every)};
    const int my_blocks[2] = {blocks_in_sight(my_pos[0], p.window, p.pool), blocks_in_sight(my_pos[1], p.window, p.pool)};

    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;             // earliest token that the first row sees
    const int pooled_rows = blocks_in_sight(last_pos, p.window, p.pool);       // pooled blocks that the last row sees
    const int pooled_tiles = (pooled_rows + BN - 1) / BN;
    const int first_block = lo / BN, last_block = last_pos / BN;
    const int* table = p.block_table + (size_t)seq * p.table_width;
    const int* ptable = p.pool_table != nullptr ? p.pool_table + (size_t)seq * p.pool_table_width : nullptr;
    const float inv_pool = p.pool > 0 ? 1.0f / (float)p.pool : 0.f;
    const int tiles = pooled_tiles + (last_block - first_block + 1);
    for (int it = 0; it < tiles; ++it) {
        const bool pooled = it < pooled_tiles;
        const int b = pooled ? it : first_block + (it - pooled_tiles);         // tile of pooled rows, or page of tokens
        const int limit = pooled ? pooled_rows : last_pos + 1;                 // rows of the source beyond this are not staged
        const int page = pooled ? ptable[b] : table[b];
        __syncthreads();                                   // the tile before is done with sk and svt
        for (int idx = tid; idx < BN * (DK / 8); idx += 128) {
            const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
            const size_t at = ((size_t)page * BN + r) * p.kv_heads + kvh;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (b * BN + r < limit) v = pooled ? piece_sum(p.pk_pool + at * p.dim, c, p.dim, inv_pool) : piece_bf16(p.k_pool + at * p.dim, c, p.dim);
            *(uint4*)(sk + r * (DK + PAD) + c) = v;
        }
        for (int idx = tid; idx < BN * (DV / 8); idx += 128) {
            // consecutive threads take consecutive keys of one piece of 8 channels: the transposed 2-byte stores below then
            // fall into different banks
            const int r = idx % BN, c = (idx / BN) * 8;
            const size_t at = ((size_t)page * BN + r) * p.kv_heads + kvh;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (b * BN + r < limit) v = pooled ? piece_sum(p.pv_pool + at * p.vdim, c, p.vdim, inv_pool) : piece_bf16(p.v_pool + at * p.vdim, c, p.vdim);
            const bf16* e = (const bf16*)&v;
#pragma unroll
            for (int i = 0; i < 8; ++i) svt[(c + i) * (BN + PAD) + r] = e[i];
        }
        __syncthreads();

        float s[BN / 8][4];
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                const bf16* kb = sk + (nt * 8 + g) * (DK + PAD) + ks * 16 + 2 * t;
                mma_16816(s[nt], qa[ks], *(const uint32_t*)kb, *(const uint32_t*)(kb + 8));
            }
        }
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = b * BN + nt * 8 + 2 * t + (e & 1), half = e >> 1;
                const int pos = my_pos[half];
                const bool seen = pos <= last_pos && (pooled ? j < my_blocks[half] : (j <= pos && (p.window <= 0 || pos - j < p.window)));
                s[nt][e] = seen ? s[nt][e] * mult[half] : -INFINITY;
                m_new[half] = fmaxf(m_new[half], s[nt][e]);
            }
        }
        float corr[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 1));
            m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 2));
            corr[half] = m_new[half] == -INFINITY ? 1.f : expf(m_run[half] - m_new[half]);
            m_run[half] = m_new[half];
            l_run[half] *= corr[half];
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        float l_add[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int half = e >> 1;
                const float w = m_new[half] == -INFINITY ? 0.f : expf(s[nt][e] - m_new[half]);
                s[nt][e] = w;
                l_add[half] += w;
            }
        }
        l_run[0] += l_add[0];
        l_run[1] += l_add[1];
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t hi[4], lw[4];
            split2(s[2 * kk][0], s[2 * kk][1], hi[0], lw[0]);
            split2(s[2 * kk][2], s[2 * kk][3], hi[1], lw[1]);
            split2(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lw[2]);
            split2(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lw[3]);
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                const bf16* vb = svt + (nt * 8 + g) * (BN + PAD) + kk * 16 + 2 * t;
                const uint32_t b0 = *(const uint32_t*)vb, b1 = *(const uint32_t*)(vb + 8);
                mma_16816(o[nt], hi, b0, b1);
                mma_16816(o[nt], lw, b0, b1);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        if (r >= n_rows) continue;
        float l = l_run[half], f = 1.f;
        if (p.sink.p != nullptr) {                          // the sink joins the denominator only
            const float sink = p.sink.at(h), big = fmaxf(m_run[half], sink);
            f = expf(m_run[half] - big);
            l = l * f + expf(sink - big);
        }
        const float inv = l > 0.f ? f / l : 0.f;
        bf16* dst = p.out + (size_t)(row0 + r) * p.heads * p.vdim + (size_t)h * p.vdim;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int c = nt * 8 + 2 * t;
            const float x = o[nt][2 * half] * inv, y = o[nt][2 * half + 1] * inv;
            if (c + 1 < p.vdim && (((uintptr_t)(dst + c)) & 3) == 0) *(uint32_t*)(dst + c) = pack2(x, y);
            else {
                if (c < p.vdim) dst[c] = __float2bfloat16_rn(x);
                if (c + 1 < p.vdim) dst[c + 1] = __float2bfloat16_rn(y);
            }
        }
    }
}

template <int DK, int DV>
int launch_prompt(const PromptArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    const size_t smem = ((size_t)(BM + BN) * (DK + PAD) + (size_t)DV * (BN + PAD)) * sizeof(bf16);
    static bool set = false;
    if (!set) {
        FR_CUDA(cudaFuncSetAttribute(prompt_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    const dim3 grid((max_q_len + BM - 1) / BM, p.heads, n_seqs);
    FR_CUDA(fr_launch(prompt_kernel<DK, DV>, grid, dim3(128), smem, stream, p));
    FR_CHECK_LAUNCH("attention_pooled prompt");
    return FR_OK;
}

template <int DK>
int prompt_by_value_size(const PromptArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    if (p.vdim <= 32) return launch_prompt<DK, 32>(p, n_seqs, max_q_len, stream);
    if (p.vdim <= 64) return launch_prompt<DK, 64>(p, n_seqs, max_q_len, stream);
    return launch_prompt<DK, 128>(p, n_seqs, max_q_len, stream);
}

int check_shape(int heads, int kv_heads, int dim, int vdim, int window, int pool, int page) {
    if (page != PAGE_ROWS) FR_REFUSE("attention_pooled: pages of %d positions (64)", page);
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) FR_REFUSE("attention_pooled: %d heads cannot share %d key/value heads", heads, kv_heads);
    if (dim <= 0 || dim > 256 || vdim <= 0 || vdim > 256) FR_REFUSE("attention_pooled: head sizes %d and %d (1 to 256)", dim, vdim);
    if (window < 0 || pool < 0 || (pool > 0 && window == 0)) FR_REFUSE("attention_pooled: window %d, pooled blocks of %d (blocks need a window)", window, pool);
    return FR_OK;
}

}  // namespace

// proj [rows][ld] of `dtype`: q heads at q_off, k heads at k_off, v heads at v_off (v_pool null: the values are the keys and
// nothing is read at v_off).  q_norm / k_norm [dim] of norm_dtype (null: no norm); freq [rot / 2] (null: no rotation).
// write 0: the cache is left alone (queries only).
FR_EXPORT int attention_pooled_prepare(void* proj, int ld, int q_off, int k_off, int v_off, const void* q_norm, const void* k_norm,
                                       int norm_dtype, float eps, const float* freq, float rot_mult, int rot, void* k_pool, void* v_pool,
                                       const int* block_table, int table_width, int page, const int* row_seq, const int* row_pos, int rows,
                                       int heads, int kv_heads, int dim, int vdim, int write, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    const int rc = check_shape(heads, kv_heads, dim, vdim, 0, 0, page);
    if (rc != FR_OK) return rc;
    if (freq != nullptr && (rot <= 0 || rot % 2 || rot > dim)) FR_REFUSE("attention_pooled: %d rotated numbers in heads of %d", rot, dim);
    PrepArgs p;
    p.proj = proj; p.q_norm = FrVec{q_norm, norm_dtype}; p.k_norm = FrVec{k_norm, norm_dtype}; p.freq = freq; p.k_pool = k_pool; p.v_pool = v_pool;
    p.block_table = block_table; p.row_seq = row_seq; p.row_pos = row_pos; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
    p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.rot = rot; p.table_width = table_width; p.rows = rows; p.write = write;
    p.eps = eps; p.rot_mult = rot_mult;
    const long long items = (long long)rows * (heads + 2 * kv_heads);
    const dim3 grid((unsigned)((items + 3) / 4));
    if (dtype == FR_F32) FR_CUDA(fr_launch(prepare_kernel<float>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(prepare_kernel<bf16>, grid, dim3(128), 0, stream, p));
    else FR_REFUSE("attention_pooled: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("attention_pooled prepare");
    return FR_OK;
}

// After prepare: the pooled rows of the blocks that the step's tokens belong to take the step's keys and values.
FR_EXPORT int attention_pooled_pool(const void* k_pool, const void* v_pool, float* pk_pool, float* pv_pool, const int* block_table,
                                    int table_width, const int* pool_table, int pool_table_width, int page, const int* seq_qlen,
                                    const int* seq_pos0, int n_seqs, int max_q_len, int kv_heads, int dim, int vdim, int pool, int dtype,
                                    cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return FR_OK;
    if (pool <= 0 || page != PAGE_ROWS) FR_REFUSE("attention_pooled: blocks of %d tokens, pages of %d", pool, page);
    PoolArgs p;
    p.k_pool = k_pool; p.v_pool = v_pool; p.pk_pool = pk_pool; p.pv_pool = pv_pool; p.block_table = block_table; p.pool_table = pool_table;
    p.seq_qlen = seq_qlen; p.seq_pos0 = seq_pos0; p.table_width = table_width; p.pool_table_width = pool_table_width; p.kv_heads = kv_heads;
    p.dim = dim; p.vdim = vdim; p.pool = pool;
    const dim3 grid(n_seqs, (max_q_len + pool - 1) / pool + 1, (kv_heads * (dim + vdim) + 127) / 128);
    if (grid.y > 65535 || grid.z > 65535) FR_REFUSE("attention_pooled: %d blocks of tokens in a step, %d channels", (int)grid.y, kv_heads * (dim + vdim));
    if (dtype == FR_F32) FR_CUDA(fr_launch(pool_kernel<float>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(pool_kernel<bf16>, grid, dim3(128), 0, stream, p));
    else FR_REFUSE("attention_pooled: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("attention_pooled pool");
    return FR_OK;
}

FR_EXPORT long long attention_pooled_scratch_floats(int rows, int heads, int vdim, int splits) {
    return (long long)rows * heads * (splits < 1 ? 1 : splits) * (vdim + 2);
}

// q [rows][q_stride] and out [rows][heads * vdim] of `dtype`, like the token pools; the pooled pools are fp32 sums (null with
// pool 0).  sink [heads] of sink_dtype (null: none).  temp_every 0: no query multiplier.
FR_EXPORT int attention_pooled_rows(const void* q, int q_stride, int q_off, void* out, const void* k_pool, const void* v_pool,
                                    const float* pk_pool, const float* pv_pool, const int* block_table, int table_width,
                                    const int* pool_table, int pool_table_width, int page, const int* row_seq, const int* row_pos, int rows,
                                    int heads, int kv_heads, int dim, int vdim, int window, int pool, float scale, float temp_coef,
                                    int temp_every, const void* sink, int sink_dtype, int splits, float* scratch, int dtype,
                                    cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    const int rc = check_shape(heads, kv_heads, dim, vdim, window, pool, page);
    if (rc != FR_OK) return rc;
    if (splits < 1 || splits > 65535 || scratch == nullptr) FR_REFUSE("attention_pooled: %d splits, scratch %p", splits, (void*)scratch);
    if (pool > 0 && (pk_pool == nullptr || pv_pool == nullptr || pool_table == nullptr)) FR_REFUSE("attention_pooled: pooled blocks without their pools");
    RowArgs p;
    p.q = q; p.out = out; p.k_pool = k_pool; p.v_pool = v_pool; p.pk_pool = pk_pool; p.pv_pool = pv_pool; p.block_table = block_table;
    p.pool_table = pool_table; p.row_seq = row_seq; p.row_pos = row_pos; p.sink = FrVec{sink, sink_dtype}; p.part = scratch;
    p.table_width = table_width; p.pool_table_width = pool_table_width; p.rows = rows; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim;
    p.vdim = vdim; p.q_stride = q_stride; p.q_off = q_off; p.window = window; p.pool = pool; p.splits = splits; p.temp_every = temp_every;
    p.scale = scale; p.temp_coef = temp_coef;
    const int items = rows * heads;
    const dim3 grid((items + 3) / 4, splits), mgrid((items + 3) / 4);
    if (dtype == FR_F32) {
        FR_CUDA(fr_launch(rows_kernel<float>, grid, dim3(128), 0, stream, p));
        FR_CUDA(fr_launch(rows_merge_kernel<float>, mgrid, dim3(128), 0, stream, p));
    } else if (dtype == FR_BF16) {
        FR_CUDA(fr_launch(rows_kernel<bf16>, grid, dim3(128), 0, stream, p));
        FR_CUDA(fr_launch(rows_merge_kernel<bf16>, mgrid, dim3(128), 0, stream, p));
    } else {
        FR_REFUSE("attention_pooled: unknown dtype %d", dtype);
    }
    FR_CHECK_LAUNCH("attention_pooled rows");
    return FR_OK;
}

// 1 if the tensor-core prompt kernel takes these sizes (bf16 only)
FR_EXPORT int attention_pooled_prompt_fits(int dim, int vdim, int page) { return dim >= 1 && dim <= 128 && vdim >= 1 && vdim <= 128 && page == PAGE_ROWS; }

FR_EXPORT int attention_pooled_prompt(const void* q, int q_stride, int q_off, void* out, const void* k_pool, const void* v_pool,
                                      const float* pk_pool, const float* pv_pool, const int* block_table, int table_width,
                                      const int* pool_table, int pool_table_width, int page, const int* seq_start, const int* seq_qlen,
                                      const int* seq_pos0, int n_seqs, int max_q_len, int heads, int kv_heads, int dim, int vdim, int window,
                                      int pool, float scale, float temp_coef, int temp_every, const void* sink, int sink_dtype,
                                      cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return FR_OK;
    const int rc = check_shape(heads, kv_heads, dim, vdim, window, pool, page);
    if (rc != FR_OK) return rc;
    if (!attention_pooled_prompt_fits(dim, vdim, page)) FR_REFUSE("attention_pooled prompt: head sizes %d and %d (1 to 128)", dim, vdim);
    if (n_seqs > 65535 || heads > 65535) FR_REFUSE("attention_pooled prompt: %d sequences, %d heads", n_seqs, heads);
    if (pool > 0 && (pk_pool == nullptr || pv_pool == nullptr || pool_table == nullptr)) FR_REFUSE("attention_pooled: pooled blocks without their pools");
    PromptArgs p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool; p.pk_pool = pk_pool; p.pv_pool = pv_pool;
    p.block_table = block_table; p.pool_table = pool_table; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_pos0 = seq_pos0;
    p.sink = FrVec{sink, sink_dtype}; p.table_width = table_width; p.pool_table_width = pool_table_width; p.q_stride = q_stride; p.q_off = q_off;
    p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.window = window; p.pool = pool; p.temp_every = temp_every;
    p.scale = scale; p.temp_coef = temp_coef;
    if (dim <= 32) return prompt_by_value_size<32>(p, n_seqs, max_q_len, stream);
    if (dim <= 64) return prompt_by_value_size<64>(p, n_seqs, max_q_len, stream);
    return prompt_by_value_size<128>(p, n_seqs, max_q_len, stream);
}
