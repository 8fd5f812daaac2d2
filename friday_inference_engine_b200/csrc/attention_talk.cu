// Softmax attention whose heads talk to each other before the softmax, over the paged cache.
//
// For a query at position i and a key at position j of its sequence, i - window < j <= i:
//
//   raw_g(i, j)   = (q_g(i) . k_kv(g)(j)) * scale - slope_g * (i - j)          every head g, kv(g) = g / (heads / kv heads)
//   mixed_h(i, j) = sum_g talk[h][g] * raw_g(i, j)                             the heads' scores mixed by a matrix
//   out_h(i)      = sum_j softmax_j(mixed_h(i, .))[j] * v_kv(h)(j)   (* sigmoid(gate_h(i)) element by element, if given)
//
// A head's softmax needs every head's score of the same (i, j), so the work is cut across the keys and not across the
// heads: `scores` computes the raw scores of ALL heads for a block of keys, mixes them and writes the mixed scores
// [row][head][slot] (slot t of a row at position i is the key j = max(0, i - window + 1) + t); `values` runs each
// head's softmax over its slots and multiplies with the values.  Scores, the mixing, the softmax and its weights are
// fp32 in both dtypes; keys, values and queries are read in the dtype they are stored in.
//
//   store    keys and values of the step's rows go to their cache rows; values may first be blended with rows that
//            another layer left for the same tokens, v <- (1 - lambda) v + lambda v_first (the blended rows are what is
//            kept), and a layer may leave its values for later layers
//   scores   CUDA cores: a block per (row, 128 keys), a thread per key, the key tile staged 32 channels at a time
//   values   CUDA cores: a block per (row, kv head); a warp per head finds maximum and sum, then all threads walk the
//            keys with the weights of up to four heads in shared memory, a value channel (or two) per thread
//   scores_mma / values_mma   bfloat16 prompts: the same two steps on the tensor cores (mma.sync.m16n8k16), 16 rows of a
//            sequence x 64 keys per block; the mixing happens in the accumulators' registers, the weights enter the
//            second product as two bf16 numbers each (head + remainder), which keeps them 32-bit in effect
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* attention_talk_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int KT = 128;            // keys per block of the CUDA-core score kernel
constexpr int DC = 32;             // channels staged at a time
constexpr int HC = 4;              // heads whose weights the value kernel holds at a time

// ------------------------------------------------------------------ store
template <typename T>
__global__ void talk_store_kernel(T* __restrict__ src, int ld, int k_off, int v_off, int nkv, int kd, int vd,
                                  const int* __restrict__ row_seq, const int* __restrict__ row_pos, T* __restrict__ k_pool,
                                  T* __restrict__ v_pool, const int* __restrict__ block_table, int table_width, int page,
                                  const T* __restrict__ first_in, FrVec lambda, T* __restrict__ first_out) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = row_pos[row];
    const int pg = block_table[(size_t)seq * table_width + pos / page];
    const size_t at = (size_t)pg * page + pos % page;
    T* s = src + (size_t)row * ld;
    T* kd_ = k_pool + at * nkv * kd;
    T* vd_ = v_pool + at * nkv * vd;
    for (int i = threadIdx.x; i < nkv * kd; i += blockDim.x) kd_[i] = s[k_off + i];
    const float lam = first_in != nullptr ? lambda.at(0) : 0.f;
    for (int i = threadIdx.x; i < nkv * vd; i += blockDim.x) {
        T v = s[v_off + i];
        if (first_in != nullptr) {
            const float a = fr_load(&v), b = fr_load(first_in + (size_t)row * nkv * vd + i);
            fr_store(&v, (1.0f - lam) * a + lam * b);
        }
        vd_[i] = v;
        if (first_out != nullptr) first_out[(size_t)row * nkv * vd + i] = v;
    }
}

// ------------------------------------------------------------------ scores, CUDA cores
struct ScoreArgs {
    const void* q;
    int q_ld;
    const void* k_pool;
    const int* table;
    int table_width, page;
    const int* row_seq;
    const int* row_pos;
    int heads, kv_heads, dim, window, stride;
    float scale;
    const float* slopes;        // [heads] or null
    FrVec talk;                 // [heads][heads] or null
    float* out;                 // [rows][heads][stride]
};

template <typename T>
__global__ void __launch_bounds__(KT) talk_scores_kernel(ScoreArgs p) {
    extern __shared__ float sm[];
    const int H = p.heads, G = p.kv_heads, dim = p.dim, per = H / G;
    float* qs = sm;                         // [H][dim]
    float* ss = qs + (size_t)H * dim;       // [H][KT]
    float* kt = ss + (size_t)H * KT;        // [KT][DC + 1]
    float* tk = kt + KT * (DC + 1);         // [H][H]
    const int row = blockIdx.y, tid = threadIdx.x;
    const int seq = p.row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    const int j0 = max(0, pos - p.window + 1), n = pos - j0 + 1;
    const int t0 = blockIdx.x * KT;
    if (t0 >= n) return;
    const T* q = (const T*)p.q + (size_t)row * p.q_ld;
    for (int i = tid; i < H * dim; i += KT) qs[i] = fr_load(q + i);
    if (p.talk.p != nullptr)
        for (int i = tid; i < H * H; i += KT) tk[i] = p.talk.at(i);
    const int* tab = p.table + (size_t)seq * p.table_width;
    const T* kp = (const T*)p.k_pool;
    const int t = t0 + tid;
    const float dist = (float)(pos - (j0 + t));
    for (int c = 0; c < G; ++c) {
        for (int hc = 0; hc < per; hc += 8) {
            float acc[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) acc[a] = 0.f;
            for (int d0 = 0; d0 < dim; d0 += DC) {
                __syncthreads();
                for (int idx = tid; idx < KT * DC; idx += KT) {
                    const int kk = idx / DC, d = idx % DC;
                    float v = 0.f;
                    if (t0 + kk < n && d0 + d < dim) {
                        const int j = j0 + t0 + kk;
                        const size_t at = (size_t)tab[j / p.page] * p.page + j % p.page;
                        v = fr_load(kp + (at * G + c) * dim + d0 + d);
                    }
                    kt[kk * (DC + 1) + d] = v;
                }
                __syncthreads();
                const int dn = min(DC, dim - d0);
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    if (hc + a < per) {
                        const float* qh = qs + (size_t)(c * per + hc + a) * dim + d0;
                        float s = acc[a];
                        for (int d = 0; d < dn; ++d) s = fmaf(qh[d], kt[tid * (DC + 1) + d], s);
                        acc[a] = s;
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                if (hc + a < per) {
                    const int h = c * per + hc + a;
                    float s = acc[a] * p.scale;
                    if (p.slopes != nullptr) s -= p.slopes[h] * dist;
                    ss[h * KT + tid] = s;
                }
            }
        }
    }
    __syncthreads();
    if (t >= n) return;
    float* o = p.out + (size_t)row * H * p.stride + t;
    for (int h = 0; h < H; ++h) {
        float s;
        if (p.talk.p != nullptr) {
            s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(tk[h * H + g], ss[g * KT + tid], s);
        } else {
            s = ss[h * KT + tid];
        }
        o[(size_t)h * p.stride] = s;
    }
}

// ------------------------------------------------------------------ softmax and values, CUDA cores
struct ValueArgs {
    const float* scores;        // [rows][heads][stride]
    const void* v_pool;
    const int* table;
    int table_width, page;
    const int* row_seq;
    const int* row_pos;
    int heads, kv_heads, vdim, window, stride;
    const void* gate;           // [rows][gate_ld], head h's gates at h * vdim; or null
    int gate_ld;
    void* out;                  // [rows][heads * vdim]
};

constexpr int VK = 256;            // keys whose weights are held at a time

template <typename T>
__global__ void __launch_bounds__(128) talk_values_kernel(ValueArgs p) {
    __shared__ float w[HC][VK];
    __shared__ float top[HC], inv[HC];
    const int H = p.heads, G = p.kv_heads, vd = p.vdim, per = H / G;
    const int row = blockIdx.x, c = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    const int j0 = max(0, pos - p.window + 1), n = pos - j0 + 1;
    const int* tab = p.table + (size_t)seq * p.table_width;
    const T* vp = (const T*)p.v_pool;
    for (int hc = 0; hc < per; hc += HC) {
        const int nh = min(HC, per - hc);
        __syncthreads();
        if (warp < nh) {                    // a warp per head: maximum, then the sum of the exponentials
            const float* s = p.scores + ((size_t)row * H + c * per + hc + warp) * p.stride;
            float m = -INFINITY;
            for (int t = lane; t < n; t += 32) m = fmaxf(m, s[t]);
            m = fr_warp_max(m);
            float sum = 0.f;
            for (int t = lane; t < n; t += 32) sum += expf(s[t] - m);
            sum = fr_warp_sum(sum);
            if (lane == 0) {
                top[warp] = m;
                inv[warp] = 1.0f / sum;
            }
        }
        for (int d0 = 0; d0 < vd; d0 += 256) {
            float acc[HC][2];
#pragma unroll
            for (int a = 0; a < HC; ++a) acc[a][0] = acc[a][1] = 0.f;
            const int da = d0 + tid, db = d0 + 128 + tid;
            for (int k0 = 0; k0 < n; k0 += VK) {
                const int kn = min(VK, n - k0);
                __syncthreads();
                if (warp < nh) {
                    const float* s = p.scores + ((size_t)row * H + c * per + hc + warp) * p.stride + k0;
                    const float m = top[warp], r = inv[warp];
                    for (int t = lane; t < kn; t += 32) w[warp][t] = expf(s[t] - m) * r;
                }
                __syncthreads();
                for (int t = 0; t < kn; ++t) {
                    const int j = j0 + k0 + t;
                    const size_t at = (size_t)tab[j / p.page] * p.page + j % p.page;
                    const T* vr = vp + (at * G + c) * vd;
                    const float va = da < vd ? fr_load(vr + da) : 0.f;
                    const float vb = db < vd ? fr_load(vr + db) : 0.f;
#pragma unroll
                    for (int a = 0; a < HC; ++a) {
                        if (a < nh) {
                            const float x = w[a][t];
                            acc[a][0] = fmaf(x, va, acc[a][0]);
                            acc[a][1] = fmaf(x, vb, acc[a][1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < HC; ++a) {
                if (a < nh) {
                    const int h = c * per + hc + a;
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int d = u == 0 ? da : db;
                        if (d < vd) {
                            float o = acc[a][u];
                            if (p.gate != nullptr) {
                                const float g = fr_load((const T*)p.gate + (size_t)row * p.gate_ld + (size_t)h * vd + d);
                                o *= 1.0f / (1.0f + expf(-g));
                            }
                            fr_store((T*)p.out + (size_t)row * H * vd + (size_t)h * vd + d, o);
                        }
                    }
                }
            }
        }
    }
}

}  // namespace

// Keys [kv_heads][dim] at column k_off and values [kv_heads][vdim] at column v_off of every row of src go to the cache rows of
// (row_seq, row_pos).  first_in (or null): rows [n_rows][kv_heads * vdim] that the values are blended with, lambda a single
// number; the blended values also replace the row's own in src.  first_out (or null) receives the values as stored.
FR_EXPORT int attention_talk_store(void* src, int ld, int k_off, int v_off, int nkv, int kd, int vd, const int* row_seq,
                                   const int* row_pos, void* k_pool, void* v_pool, const int* block_table, int table_width, int page,
                                   int n_rows, int dtype, const void* first_in, const void* lambda, int lambda_dtype, void* first_out,
                                   cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (k_pool == nullptr || v_pool == nullptr || block_table == nullptr) FR_REFUSE("talk store: no cache to write to");
    if (first_in != nullptr && lambda == nullptr) FR_REFUSE("talk store: blending needs its weight");
    const FrVec lam{lambda, lambda_dtype};
    if (dtype == FR_F32)
        FR_CUDA(fr_launch(talk_store_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (float*)src, ld, k_off, v_off, nkv, kd, vd, row_seq,
                          row_pos, (float*)k_pool, (float*)v_pool, block_table, table_width, page, (const float*)first_in, lam,
                          (float*)first_out));
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(talk_store_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (bf16*)src, ld, k_off, v_off, nkv, kd, vd, row_seq,
                          row_pos, (bf16*)k_pool, (bf16*)v_pool, block_table, table_width, page, (const bf16*)first_in, lam,
                          (bf16*)first_out));
    else
        FR_REFUSE("talk store: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("talk store");
    return FR_OK;
}

// Floats that `scores` writes and `values` reads for n_rows rows: [rows][heads][stride], stride = the most keys a row sees,
// rounded up to 4.
FR_EXPORT long long attention_talk_stride(int window, int max_kv_len) {
    const int span = window > 0 && window < max_kv_len ? window : max_kv_len;
    return (long long)((span + 3) / 4 * 4);
}

FR_EXPORT int attention_talk_scores(const void* q, int q_ld, const void* k_pool, const int* table, int table_width, int page,
                                    const int* row_seq, const int* row_pos, int n_rows, int heads, int kv_heads, int dim, int window,
                                    int max_kv_len, float scale, const float* slopes, const void* talk, int talk_dtype, float* out,
                                    int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0) FR_REFUSE("talk scores: %d heads on %d key heads of %d", heads, kv_heads, dim);
    if (window <= 0) window = max_kv_len;
    ScoreArgs p;
    p.q = q; p.q_ld = q_ld; p.k_pool = k_pool; p.table = table; p.table_width = table_width; p.page = page;
    p.row_seq = row_seq; p.row_pos = row_pos; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.window = window;
    p.stride = (int)attention_talk_stride(window, max_kv_len);
    p.scale = scale; p.slopes = slopes; p.talk = FrVec{talk, talk_dtype}; p.out = out;
    const size_t smem = ((size_t)heads * dim + (size_t)heads * KT + KT * (DC + 1) + (size_t)heads * heads) * sizeof(float);
    if (smem > 200 * 1024) FR_REFUSE("talk scores: %d heads of %d need %zu bytes of shared memory", heads, dim, smem);
    const dim3 grid((unsigned)((p.stride + KT - 1) / KT), (unsigned)n_rows);
    if (dtype == FR_F32) {
        FR_CUDA(cudaFuncSetAttribute(talk_scores_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(talk_scores_kernel<float>, grid, dim3(KT), smem, stream, p));
    } else if (dtype == FR_BF16) {
        FR_CUDA(cudaFuncSetAttribute(talk_scores_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(talk_scores_kernel<bf16>, grid, dim3(KT), smem, stream, p));
    } else {
        FR_REFUSE("talk scores: unknown dtype %d", dtype);
    }
    FR_CHECK_LAUNCH("talk scores");
    return FR_OK;
}

FR_EXPORT int attention_talk_values(const float* scores, const void* v_pool, const int* table, int table_width, int page,
                                    const int* row_seq, const int* row_pos, int n_rows, int heads, int kv_heads, int vdim, int window,
                                    int max_kv_len, const void* gate, int gate_ld, void* out, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || vdim <= 0) FR_REFUSE("talk values: %d heads on %d value heads of %d", heads, kv_heads, vdim);
    if (window <= 0) window = max_kv_len;
    ValueArgs p;
    p.scores = scores; p.v_pool = v_pool; p.table = table; p.table_width = table_width; p.page = page; p.row_seq = row_seq;
    p.row_pos = row_pos; p.heads = heads; p.kv_heads = kv_heads; p.vdim = vdim; p.window = window;
    p.stride = (int)attention_talk_stride(window, max_kv_len);
    p.gate = gate; p.gate_ld = gate_ld; p.out = out;
    const dim3 grid((unsigned)n_rows, (unsigned)kv_heads);
    if (dtype == FR_F32) FR_CUDA(fr_launch(talk_values_kernel<float>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(talk_values_kernel<bf16>, grid, dim3(128), 0, stream, p));
    else FR_REFUSE("talk values: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("talk values");
    return FR_OK;
}
