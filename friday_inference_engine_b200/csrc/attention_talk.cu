// Softmax attention whose heads talk to each other before the softmax, over the paged cache.
//
// For a query at position i and a key at position j of its sequence, i - window < j <= i:
//
//   raw_g(i, j)   = (q_g(i) . k_kv(g)(j)) * scale - slope_g * (i - j)          every head g, kv(g) = g / (heads / kv heads)
//   mixed_h(i, j) = sum_g talk[h][g] * raw_g(i, j)                             the heads' scores mixed by a matrix
//   out_h(i)      = sum_j softmax_j(mixed_h(i, .))[j] * v_kv(h)(j)   (* sigmoid(gate_h(i)) element by element, if given)
//
// A head's softmax needs every head's score of the same (i, j), so the work is cut across the keys and not across the
// heads: a block owns some keys of a row (or of 16 rows) and ALL heads, computes the raw scores, and mixes them.  Scores,
// the mixing, the softmax and its weights are fp32 in both dtypes; keys, values and queries are read in the dtype they are
// stored in.
//
//   store    keys and values of the step's rows go to their cache rows; values may first be blended with rows that
//            another layer left for the same tokens, v <- (1 - lambda) v + lambda v_first (the blended rows are what is
//            kept), and a layer may leave its values for later layers
//   staged   single rows and everything in float32, CUDA cores: a block per (row, 16, 32 or 64 keys) brings its keys and
//            values into shared memory with all copies in flight at once, then scores of all heads, the mixing, each
//            head's maximum and sum, and the weighted values of the block's keys; `split` is the same block reading the
//            cache as it goes, for rows of keys or values that are not whole 16-byte pieces
//   merge    a block per (head, row) joins what the row's blocks left (maximum / sum rule) and applies the gate
//   prompt_scores / prompt_values   bfloat16 prompts on the tensor cores (mma.sync.m16n8k16): 16 rows of a sequence x 64
//            keys x all heads per block, the mixing in the accumulators' registers, the mixed scores through memory once
//            ([row][head][keys in sight] floats); then 64 rows x one head per block run the softmax block of keys by
//            block of keys and enter the weights into the second product as two bf16 numbers each (head + remainder),
//            which keeps them 32-bit in effect
#include <math.h>
#include <stdlib.h>

#include "common.cuh"

FR_EXPORT const char* attention_talk_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int KS = 64;             // keys per block of the CUDA-core kernel
constexpr int HC = 4;              // heads whose weighted values a thread sums at a time
constexpr int KS_MIN = 16;         // fewest keys per block of the staged kernel

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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

// ------------------------------------------------------------------ a row's keys in splits, CUDA cores
struct SplitArgs {
    const void* q;
    int q_ld;
    const void* k_pool;
    const void* v_pool;
    const int* table;
    int table_width, page;
    const int* row_seq;
    const int* row_pos;
    int heads, kv_heads, dim, vdim, window, splits;
    int ks;                     // keys per block
    float scale;
    const float* slopes;        // [heads] or null
    FrVec talk;                 // [heads][heads] or null
    float* part;                // [rows][splits][heads][vdim + 2]: weighted values (unnormalised), maximum, sum
};

template <typename T, int VEC>
struct Chunk;                   // VEC neighbouring channels of a key as floats
template <typename T>
struct Chunk<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float (&f)[1]) { f[0] = fr_load(p); }
};
template <>
struct Chunk<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = *(const float4*)p;
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <>
struct Chunk<bf16, 8> {
    static __device__ __forceinline__ void load(const bf16* p, float (&f)[8]) {
        const uint4 v = *(const uint4*)p;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// A block owns KS consecutive keys of one row's window and every head.  Four neighbouring lanes share a key: each takes
// every fourth chunk of VEC channels, two shuffles sum the parts.  The raw scores of all heads are mixed in shared memory,
// each head's maximum and sum over the block's keys are found by a warp, and the weighted values of the block's keys are
// summed with a thread per value channel.  What the block leaves is merged with the other blocks' by `talk_merge_kernel`.
template <typename T, int VEC>
__global__ void __launch_bounds__(128) talk_split_kernel(SplitArgs p) {
    extern __shared__ __align__(16) float sm[];
    const int H = p.heads, G = p.kv_heads, dim = p.dim, vd = p.vdim, per = H / G;
    int* koff = (int*)sm;                               // [KS] cache row of each key
    float* ms = sm + KS;                                // [H][KS] mixed scores, then weights
    float* ss = ms + (size_t)H * KS;                    // [H][KS] raw scores
    float* qs = ss + (size_t)H * KS;                    // [H][dim]
    float* tk = qs + (size_t)H * dim;                   // [H][H]
    float* stat = tk + (size_t)H * H;                   // [H][2]
    const int row = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    const int j0 = max(0, pos - p.window + 1), n = pos - j0 + 1;
    const int t0 = blockIdx.x * KS;
    if (t0 >= n) return;
    const int kn = min(KS, n - t0);
    const T* q = (const T*)p.q + (size_t)row * p.q_ld;
    for (int i = tid; i < H * dim; i += 128) qs[i] = fr_load(q + i);
    if (p.talk.p != nullptr)
        for (int i = tid; i < H * H; i += 128) tk[i] = p.talk.at(i);
    const int* tab = p.table + (size_t)seq * p.table_width;
    for (int t = tid; t < KS; t += 128) {
        const int j = j0 + t0 + min(t, kn - 1);
        koff[t] = tab[j / p.page] * p.page + j % p.page;
    }
    __syncthreads();
    const T* kp = (const T*)p.k_pool;
    const int c = tid & 3, nchunks = dim / VEC;
    for (int pass = 0; pass < KS / 32; ++pass) {
        const int t = pass * 32 + (tid >> 2);
        const float dist = (float)(pos - (j0 + t0 + t));
        const T* krow = kp + (size_t)koff[t] * G * dim;
        for (int g = 0; g < G; ++g) {
            for (int hc = 0; hc < per; hc += 8) {
                float acc[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) acc[a] = 0.f;
                for (int ci = c; ci < nchunks; ci += 4) {
                    float kf[VEC];
                    Chunk<T, VEC>::load(krow + (size_t)g * dim + ci * VEC, kf);
#pragma unroll
                    for (int a = 0; a < 8; ++a) {
                        if (hc + a < per) {
                            const float* qh = qs + (size_t)(g * per + hc + a) * dim + ci * VEC;
                            float s = acc[a];
                            if (VEC % 4 == 0) {                 // 16-byte pieces: dim is a multiple of VEC
#pragma unroll
                                for (int e = 0; e < VEC / 4; ++e) {
                                    const float4 qv = *(const float4*)(qh + 4 * e);
                                    s = fmaf(qv.x, kf[4 * e], fmaf(qv.y, kf[4 * e + 1], fmaf(qv.z, kf[4 * e + 2], fmaf(qv.w, kf[4 * e + 3], s))));
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < VEC; ++e) s = fmaf(qh[e], kf[e], s);
                            }
                            acc[a] = s;
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    if (hc + a < per) {
                        float s = acc[a];
                        s += __shfl_xor_sync(0xffffffffu, s, 1);
                        s += __shfl_xor_sync(0xffffffffu, s, 2);
                        if (c == 0) {
                            const int h = g * per + hc + a;
                            s *= p.scale;
                            if (p.slopes != nullptr) s -= p.slopes[h] * dist;
                            ss[h * KS + t] = s;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < H * KS; idx += 128) {
        const int h = idx / KS, t = idx - h * KS;
        float s;
        if (p.talk.p != nullptr) {
            s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(tk[h * H + g], ss[g * KS + t], s);
        } else {
            s = ss[idx];
        }
        ms[idx] = t < kn ? s : -INFINITY;
    }
    __syncthreads();
    for (int h = warp; h < H; h += 4) {
        float* s = ms + (size_t)h * KS;
        float m = -INFINITY;
        for (int t = lane; t < KS; t += 32) m = fmaxf(m, s[t]);
        m = fr_warp_max(m);
        float sum = 0.f;
        for (int t = lane; t < KS; t += 32) {
            const float w = expf(s[t] - m);            // keys beyond the row's last: exp(-inf) = 0
            s[t] = w;
            sum += w;
        }
        sum = fr_warp_sum(sum);
        if (lane == 0) {
            stat[2 * h] = m;
            stat[2 * h + 1] = sum;
        }
    }
    __syncthreads();
    const T* vp = (const T*)p.v_pool;
    float* part = p.part + ((size_t)row * p.splits + blockIdx.x) * H * (vd + 2);
    const int kn4 = (kn + 3) & ~3;                      // the weights past kn are zero, their rows the last key's
    for (int d = tid; d < vd; d += 128) {
        for (int g = 0; g < G; ++g) {
            for (int hc = 0; hc < per; hc += HC) {
                float acc[HC];
#pragma unroll
                for (int a = 0; a < HC; ++a) acc[a] = 0.f;
                for (int t = 0; t < kn4; t += 4) {
                    const int4 at = *(const int4*)(koff + t);
                    const float v0 = fr_load(vp + ((size_t)at.x * G + g) * vd + d);
                    const float v1 = fr_load(vp + ((size_t)at.y * G + g) * vd + d);
                    const float v2 = fr_load(vp + ((size_t)at.z * G + g) * vd + d);
                    const float v3 = fr_load(vp + ((size_t)at.w * G + g) * vd + d);
#pragma unroll
                    for (int a = 0; a < HC; ++a) {
                        if (hc + a < per) {
                            const float4 w = *(const float4*)(ms + (size_t)(g * per + hc + a) * KS + t);
                            acc[a] = fmaf(w.x, v0, fmaf(w.y, v1, fmaf(w.z, v2, fmaf(w.w, v3, acc[a]))));
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < HC; ++a)
                    if (hc + a < per) part[(size_t)(g * per + hc + a) * (vd + 2) + d] = acc[a];
            }
        }
    }
    for (int h = tid; h < H; h += 128) {
        part[(size_t)h * (vd + 2) + vd] = stat[2 * h];
        part[(size_t)h * (vd + 2) + vd + 1] = stat[2 * h + 1];
    }
}

__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) {
    const float2 v = *(const float2*)p;
    a = v.x; b = v.y;
}
__device__ __forceinline__ void load_pair(const bf16* p, float& a, float& b) {
    const uint32_t v = *(const uint32_t*)p;
    a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
}

// The same block of work with the keys and values of its `ks` keys (a multiple of four, at most KS) brought into shared
// memory first: every thread issues its 16-byte copies at once, so the block's whole share of the cache is in flight
// together, and queries and the mixing matrix are read meanwhile.  256 threads: 256 / ks lanes per key (four at 64) for the scores, a
// thread per pair of value channels of a key head for the weighted values.  A key's row in shared memory is 64 bytes
// longer than its channels, so that the 16-byte reads of two neighbouring keys fall on different banks.
template <typename T>
__global__ void __launch_bounds__(256) talk_staged_kernel(SplitArgs p) {
    constexpr int VEC = 16 / (int)sizeof(T);
    extern __shared__ __align__(16) float sm[];
    const int H = p.heads, G = p.kv_heads, dim = p.dim, vd = p.vdim, per = H / G, ks = p.ks;
    const int krow_len = G * dim + 64 / (int)sizeof(T), vrow_len = G * vd;
    float* ms = sm;                                     // [H][ks] mixed scores, then weights
    float* ss = ms + (size_t)H * ks;                    // [H][ks] raw scores
    float* qs = ss + (size_t)H * ks;                    // [H][dim]
    float* tk = qs + (size_t)H * dim;                   // [H][H]
    float* stat = tk + (size_t)H * H;                   // [H][2]
    T* kt = (T*)(((uintptr_t)(stat + 2 * (size_t)H) + 15) & ~(uintptr_t)15);   // [ks][krow_len], 16-byte aligned
    T* vt = kt + (size_t)ks * krow_len;                 // [ks][vrow_len]
    const int row = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    const int j0 = max(0, pos - p.window + 1), n = pos - j0 + 1;
    const int t0 = blockIdx.x * ks;
    if (t0 >= n) return;
    const int kn = min(ks, n - t0);
    const int* tab = p.table + (size_t)seq * p.table_width;
    {
        const T* kp = (const T*)p.k_pool;
        const T* vp = (const T*)p.v_pool;
        const int kc = G * dim / VEC, vc = G * vd / VEC;            // 16-byte pieces of a key's and of a value's row
        for (int i = tid; i < ks * (kc + vc); i += 256) {
            const int t = i / (kc + vc), c = i - t * (kc + vc);
            const int j = j0 + t0 + min(t, kn - 1);                  // slots past the row's last key repeat it; their weights are 0
            const size_t at = (size_t)tab[j / p.page] * p.page + j % p.page;
            if (c < kc) cp_async16(kt + (size_t)t * krow_len + c * VEC, kp + at * G * dim + c * VEC, 16);
            else cp_async16(vt + (size_t)t * vrow_len + (c - kc) * VEC, vp + at * G * vd + (c - kc) * VEC, 16);
        }
        cp_commit();
    }
    const T* q = (const T*)p.q + (size_t)row * p.q_ld;
    for (int i = tid; i < H * dim; i += 256) qs[i] = fr_load(q + i);
    if (p.talk.p != nullptr)
        for (int i = tid; i < H * H; i += 256) tk[i] = p.talk.at(i);
    cp_wait<0>();
    __syncthreads();
    const int lpk = ks >= 64 ? 4 : 256 / ks;                        // lanes that share a key: 4, 8 or 16
    const int c4 = tid % lpk, nchunks = dim / VEC;
    for (int t = tid / lpk; t < ks; t += 256 / lpk) {
        const float dist = (float)(pos - (j0 + t0 + t));
        const T* krow = kt + (size_t)t * krow_len;
        for (int g = 0; g < G; ++g) {
            for (int hc = 0; hc < per; hc += 8) {
                float acc[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) acc[a] = 0.f;
                for (int ci = c4; ci < nchunks; ci += lpk) {
                    float kf[VEC];
                    Chunk<T, VEC>::load(krow + (size_t)g * dim + ci * VEC, kf);
#pragma unroll
                    for (int a = 0; a < 8; ++a) {
                        if (hc + a < per) {
                            const float* qh = qs + (size_t)(g * per + hc + a) * dim + ci * VEC;
                            float s = acc[a];
#pragma unroll
                            for (int e = 0; e < VEC / 4; ++e) {
                                const float4 qv = *(const float4*)(qh + 4 * e);
                                s = fmaf(qv.x, kf[4 * e], fmaf(qv.y, kf[4 * e + 1], fmaf(qv.z, kf[4 * e + 2], fmaf(qv.w, kf[4 * e + 3], s))));
                            }
                            acc[a] = s;
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    if (hc + a < per) {
                        float s = acc[a];
                        for (int o = lpk >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                        if (c4 == 0) {
                            const int h = g * per + hc + a;
                            s *= p.scale;
                            if (p.slopes != nullptr) s -= p.slopes[h] * dist;
                            ss[h * ks + t] = s;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < H * ks; idx += 256) {
        const int h = idx / ks, t = idx - h * ks;
        float s;
        if (p.talk.p != nullptr) {
            s = 0.f;
            for (int g = 0; g < H; ++g) s = fmaf(tk[h * H + g], ss[g * ks + t], s);
        } else {
            s = ss[idx];
        }
        ms[idx] = t < kn ? s : -INFINITY;
    }
    __syncthreads();
    for (int h = warp; h < H; h += 8) {
        float* s = ms + (size_t)h * ks;
        float m = -INFINITY;
        for (int t = lane; t < ks; t += 32) m = fmaxf(m, s[t]);
        m = fr_warp_max(m);
        float sum = 0.f;
        for (int t = lane; t < ks; t += 32) {
            const float w = expf(s[t] - m);            // slots past the row's last key: exp(-inf) = 0
            s[t] = w;
            sum += w;
        }
        sum = fr_warp_sum(sum);
        if (lane == 0) {
            stat[2 * h] = m;
            stat[2 * h + 1] = sum;
        }
    }
    __syncthreads();
    float* part = p.part + ((size_t)row * p.splits + blockIdx.x) * H * (vd + 2);
    const int half = vd / 2;
    for (int item = tid; item < G * half; item += 256) {
        const int g = item / half, d = 2 * (item - g * half);
        const T* vcol = vt + (size_t)g * vd + d;
        for (int hc = 0; hc < per; hc += HC) {
            float a0[HC], a1[HC];
#pragma unroll
            for (int a = 0; a < HC; ++a) a0[a] = a1[a] = 0.f;
            for (int t = 0; t < ks; t += 4) {
                float x[4], y[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) load_pair(vcol + (size_t)(t + e) * vrow_len, x[e], y[e]);
#pragma unroll
                for (int a = 0; a < HC; ++a) {
                    if (hc + a < per) {
                        const float4 w = *(const float4*)(ms + (size_t)(g * per + hc + a) * ks + t);
                        a0[a] = fmaf(w.x, x[0], fmaf(w.y, x[1], fmaf(w.z, x[2], fmaf(w.w, x[3], a0[a]))));
                        a1[a] = fmaf(w.x, y[0], fmaf(w.y, y[1], fmaf(w.z, y[2], fmaf(w.w, y[3], a1[a]))));
                    }
                }
            }
#pragma unroll
            for (int a = 0; a < HC; ++a)
                if (hc + a < per) *(float2*)(part + (size_t)(g * per + hc + a) * (vd + 2) + d) = make_float2(a0[a], a1[a]);
        }
    }
    for (int h = tid; h < H; h += 256) {
        part[(size_t)h * (vd + 2) + vd] = stat[2 * h];
        part[(size_t)h * (vd + 2) + vd + 1] = stat[2 * h + 1];
    }
}

struct MergeTalkArgs {
    const float* part;          // [rows][splits][heads][vdim + 2]
    const int* row_seq;
    const int* row_pos;
    int heads, vdim, window, splits, ks;
    const void* gate;           // [rows][gate_ld], head h's gates at h * vdim; or null
    int gate_ld;
    void* out;                  // [rows][heads * vdim]
};

// out_h = sum_s o_s exp(m_s - M) / sum_s l_s exp(m_s - M) over the row's blocks of keys, times sigmoid(gate) if given.
// A block per (head, row): the blocks' factors are found once, in shared memory, then a thread per value channel sums.
template <typename T>
__global__ void __launch_bounds__(128) talk_merge_kernel(MergeTalkArgs p) {
    extern __shared__ __align__(16) float sm[];            // [splits] factors
    __shared__ float red[8];
    const int h = blockIdx.x, row = blockIdx.y, H = p.heads, vd = p.vdim, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = p.row_pos[row];
    const int n = pos - max(0, pos - p.window + 1) + 1;
    const int ns = (n + p.ks - 1) / p.ks;
    const size_t step = (size_t)H * (vd + 2);
    const float* ph = p.part + (size_t)row * p.splits * step + (size_t)h * (vd + 2);
    float big = -INFINITY;
    for (int s = tid; s < ns; s += 128) big = fmaxf(big, ph[s * step + vd]);
    big = fr_warp_max(big);
    if (lane == 0) red[warp] = big;
    __syncthreads();
    big = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float l = 0.f;
    for (int s = tid; s < ns; s += 128) {
        const float f = expf(ph[s * step + vd] - big);
        sm[s] = f;
        l = fmaf(ph[s * step + vd + 1], f, l);
    }
    l = fr_warp_sum(l);
    if (lane == 0) red[4 + warp] = l;
    __syncthreads();
    l = (red[4] + red[5]) + (red[6] + red[7]);
    const float inv = 1.0f / l;
    for (int d = tid; d < vd; d += 128) {
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        int s = 0;
        for (; s + 4 <= ns; s += 4) {
            o0 = fmaf(ph[s * step + d], sm[s], o0);
            o1 = fmaf(ph[(s + 1) * step + d], sm[s + 1], o1);
            o2 = fmaf(ph[(s + 2) * step + d], sm[s + 2], o2);
            o3 = fmaf(ph[(s + 3) * step + d], sm[s + 3], o3);
        }
        for (; s < ns; ++s) o0 = fmaf(ph[s * step + d], sm[s], o0);
        float o = ((o0 + o1) + (o2 + o3)) * inv;
        if (p.gate != nullptr) {
            const float g = fr_load((const T*)p.gate + (size_t)row * p.gate_ld + (size_t)h * vd + d);
            o *= 1.0f / (1.0f + expf(-g));
        }
        fr_store((T*)p.out + (size_t)row * H * vd + (size_t)h * vd + d, o);
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

// Floats of scratch memory that `attention_talk_rows` needs for n_rows rows: what every block of keys of a row leaves, sized
// for the smallest blocks.
static int talk_span(int window, int max_kv_len) {
    const int span = window > 0 && window < max_kv_len ? window : max_kv_len;
    return span > 0 ? span : 1;
}

FR_EXPORT long long attention_talk_scratch_floats(int n_rows, int heads, int vdim, int window, int max_kv_len) {
    return (long long)n_rows * ((talk_span(window, max_kv_len) + KS_MIN - 1) / KS_MIN) * heads * (vdim + 2);
}

template <typename T, int VEC>
static cudaError_t launch_split(const SplitArgs& p, dim3 grid, size_t smem, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(talk_split_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return fr_launch(talk_split_kernel<T, VEC>, grid, dim3(128), smem, stream, p);
}

template <typename T>
static cudaError_t launch_staged(const SplitArgs& p, dim3 grid, size_t smem, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(talk_staged_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return fr_launch(talk_staged_kernel<T>, grid, dim3(256), smem, stream, p);
}

// shared memory of the staged kernel with ks keys per block
static size_t staged_bytes(int ks, int heads, int kv_heads, int dim, int vdim, size_t esz) {
    return (2 * (size_t)heads * ks + (size_t)heads * dim + (size_t)heads * heads + 2 * (size_t)heads) * sizeof(float) + 16 +
           (size_t)ks * ((size_t)kv_heads * dim * esz + 64) + (size_t)ks * kv_heads * vdim * esz;
}

// out [n_rows][heads * vdim]: every row's attention over the keys of its window, on the CUDA cores, in two launches: blocks of
// keys, then their merge (with the gate).  q: [n_rows][q_ld], head h at h * dim; gate (or null): [n_rows][gate_ld].
// Where rows of keys and values are whole 16-byte pieces the blocks stage them in shared memory, with as many keys per
// block (64, 32 or 16) as fit there and leave about one and a half blocks per SM or more; otherwise blocks of 64 keys read
// them from the cache as they go.
FR_EXPORT int attention_talk_rows(const void* q, int q_ld, const void* k_pool, const void* v_pool, const int* table, int table_width,
                                  int page, const int* row_seq, const int* row_pos, int n_rows, int heads, int kv_heads, int dim, int vdim,
                                  int window, int max_kv_len, float scale, const float* slopes, const void* talk, int talk_dtype,
                                  const void* gate, int gate_ld, void* out, float* scratch, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0)
        FR_REFUSE("talk attention: %d heads on %d key heads of %d and %d", heads, kv_heads, dim, vdim);
    if (dtype != FR_F32 && dtype != FR_BF16) FR_REFUSE("talk attention: unknown dtype %d", dtype);
    if (window <= 0) window = max_kv_len;
    const int span = talk_span(window, max_kv_len);
    SplitArgs p;
    p.q = q; p.q_ld = q_ld; p.k_pool = k_pool; p.v_pool = v_pool; p.table = table; p.table_width = table_width; p.page = page;
    p.row_seq = row_seq; p.row_pos = row_pos; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim; p.window = window;
    p.scale = scale; p.slopes = slopes; p.talk = FrVec{talk, talk_dtype}; p.part = scratch;
    const size_t esz = dtype == FR_F32 ? 4 : 2;
    const bool k_pieces = ((uintptr_t)k_pool % 16) == 0 && ((size_t)dim * esz) % 16 == 0;
    const bool v_pieces = ((uintptr_t)v_pool % 16) == 0 && ((size_t)vdim * esz) % 16 == 0 && ((uintptr_t)scratch % 8) == 0;
    const size_t room = 200 * 1024;
    int ks = 0;
    if (k_pieces && v_pieces) {
        // FRIDAY_TALK_KEYS=16|32|64 forces the keys per block where they fit (for sweeps)
        static const int forced = [] {
            const char* e = getenv("FRIDAY_TALK_KEYS");
            const int v = e != nullptr ? atoi(e) : 0;
            return v == 16 || v == 32 || v == 64 ? v : 0;
        }();
        ks = forced > 0 ? forced : KS;
        while (ks > KS_MIN && (staged_bytes(ks, heads, kv_heads, dim, vdim, esz) > room ||
                               (forced == 0 && (long long)n_rows * ((span + ks - 1) / ks) < 222)))
            ks /= 2;
        if (staged_bytes(ks, heads, kv_heads, dim, vdim, esz) > room) ks = 0;
    }
    cudaError_t launched;
    if (ks > 0) {
        p.ks = ks;
        p.splits = (span + ks - 1) / ks;
        const dim3 grid((unsigned)p.splits, (unsigned)n_rows);
        const size_t smem = staged_bytes(ks, heads, kv_heads, dim, vdim, esz);
        launched = dtype == FR_F32 ? launch_staged<float>(p, grid, smem, stream) : launch_staged<bf16>(p, grid, smem, stream);
    } else {
        p.ks = KS;
        p.splits = (span + KS - 1) / KS;
        const dim3 grid((unsigned)p.splits, (unsigned)n_rows);
        const size_t smem = ((size_t)KS + 2 * (size_t)heads * KS + (size_t)heads * dim + (size_t)heads * heads + 2 * (size_t)heads) * sizeof(float);
        if (smem > room) FR_REFUSE("talk attention: %d heads of %d need %zu bytes of shared memory", heads, dim, smem);
        if (dtype == FR_F32) launched = k_pieces ? launch_split<float, 4>(p, grid, smem, stream) : launch_split<float, 1>(p, grid, smem, stream);
        else launched = k_pieces ? launch_split<bf16, 8>(p, grid, smem, stream) : launch_split<bf16, 1>(p, grid, smem, stream);
    }
    FR_CUDA(launched);
    FR_CHECK_LAUNCH("talk blocks");
    MergeTalkArgs m;
    m.part = scratch; m.row_seq = row_seq; m.row_pos = row_pos; m.heads = heads; m.vdim = vdim; m.window = window; m.splits = p.splits;
    m.ks = p.ks; m.gate = gate; m.gate_ld = gate_ld; m.out = out;
    const dim3 mgrid((unsigned)heads, (unsigned)n_rows);
    const size_t msm = (size_t)p.splits * sizeof(float);
    if (msm > 48 * 1024) FR_REFUSE("talk attention: %d blocks of keys per row are more than the merge takes", p.splits);
    if (dtype == FR_F32) FR_CUDA(fr_launch(talk_merge_kernel<float>, mgrid, dim3(128), msm, stream, m));
    else FR_CUDA(fr_launch(talk_merge_kernel<bf16>, mgrid, dim3(128), msm, stream, m));
    FR_CHECK_LAUNCH("talk merge");
    return FR_OK;
}

// ------------------------------------------------------------------ bfloat16 prompts on the tensor cores
// The mixed scores go through memory once, [row][head][stride] floats.  A row at position i sees the keys j0 = max(0, i -
// window + 1) .. i; slot t of its stride is the key (j0 / 64) * 64 + t, so that a block of 64 keys (a page) starts at a
// multiple of 64 slots in every row and 16-byte accesses stay aligned.
namespace {

constexpr int PB = 64;             // keys per block: a page of the cache
constexpr float LOG2E = 1.4426950408889634f;
constexpr int QR = 16;             // rows of a sequence per CTA of the score kernel

static int prompt_stride(int window, int max_kv_len) {
    const int all = (max_kv_len + PB - 1) / PB;
    const int seen = window > 0 ? (window + PB - 1) / PB + 1 : all;
    return (seen < all ? seen : all) * PB;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *(const uint32_t*)&v;
}

// head and remainder of two fp32 weights as packed bf16 pairs: w = hi + lo to 2^-17
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
    const bf16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
    const __nv_bfloat162 h = __halves2bfloat162(hx, hy);
    hi = *(const uint32_t*)&h;
    lo = pack_bf16(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

struct PromptArgs {
    const bf16* q;              // [rows][q_ld], head h at h * dim
    int q_ld;
    const bf16* k_pool;         // [pages][64][kv_heads][dim]
    const bf16* v_pool;         // [pages][64][kv_heads][vdim]
    const int* table;
    int table_width;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_pos0;
    int heads, kv_heads, dim, q_ld_s, vdim, window, stride;
    float scale;
    const float* slopes;
    FrVec talk;
    const bf16* gate;
    int gate_ld;
    bf16* out;                  // [rows][heads * vdim]
    float* mixed;               // [rows][heads][stride]
};

// 16 rows of a sequence, one block of 64 keys, every head.  The rows' queries are staged once for all heads; each of the
// eight warps owns 8 of the keys and keeps scale * q.k - slope * distance of all heads in its accumulators (m16n8k16 with
// the channels of a group of 32 dealt out so that a thread's 16-byte read of a query row and of its key are its A and B
// fragments of two steps: a product does not care in which order its channels are summed, only that A and B agree).
// The heads are then mixed in the registers, the matrix read from shared memory, and the mixed scores stored.
template <int HP>
__global__ void __launch_bounds__(256, HP <= 16 ? 2 : 1) talk_prompt_scores_kernel(PromptArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = p.heads, per = H / p.kv_heads, dim = p.dim, G = p.kv_heads;
    const int lq = p.q_ld_s;
    float* tk = (float*)smem_raw;                                   // [HP][HP]: tk[h][g] = talk[h][g], zeros beyond H
    float* sl = tk + HP * HP;                                       // [HP] slopes
    bf16* sq = (bf16*)(sl + HP);                                    // [QR][lq]
    const int seq = blockIdx.z, q0 = blockIdx.y * QR;
    const int qlen = p.seq_qlen[seq];
    if (q0 >= qlen) return;
    const int n_rows = min(QR, qlen - q0);
    const int pos0 = p.seq_pos0[seq] + q0, last_pos = pos0 + n_rows - 1;
    const int lo0 = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b = lo0 / PB + blockIdx.x;
    if (b > last_pos / PB) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t4 = lane & 3;
    for (int i = tid; i < HP * HP; i += 256) {
        const int h = i / HP, g = i - h * HP;
        tk[i] = (h < H && g < H) ? (p.talk.p != nullptr ? p.talk.at(h * H + g) : (h == g ? 1.f : 0.f)) : 0.f;
    }
    for (int i = tid; i < HP; i += 256) sl[i] = (i < H && p.slopes != nullptr) ? p.slopes[i] : 0.f;
    fr_pdl_wait();
    fr_pdl_launch();
    const int row0 = p.seq_start[seq] + q0;
    const int cpr = H * dim / 8;                                     // 16-byte pieces per row
    for (int idx = tid; idx < QR * cpr; idx += 256) {
        const int r = idx / cpr, c = (idx - r * cpr) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) v = *(const uint4*)(p.q + (size_t)(row0 + r) * p.q_ld + c);
        *(uint4*)(sq + (size_t)r * lq + c) = v;
    }
    __syncthreads();
    const int page = p.table[(size_t)seq * p.table_width + b];
    const int key = b * PB + warp * 8 + gid;                        // the key whose channels this thread reads
    const bf16* krow = p.k_pool + ((size_t)page * PB + warp * 8 + gid) * G * dim;
    const bool key_ok = key <= last_pos;
    const bf16* qa_row = sq + (size_t)gid * lq + t4 * 8;
    const bf16* qb_row = qa_row + (size_t)8 * lq;
    float acc[HP][4];
#pragma unroll
    for (int h = 0; h < HP; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
    const int nch = (dim + 31) / 32;
    for (int c = 0; c < nch; ++c) {
        const int ch = c * 32 + t4 * 8;                             // this thread's eight channels of the group
        const bool ch_ok = ch < dim;
        uint4 kf = make_uint4(0, 0, 0, 0);
        int left = 0;                                               // heads that still use the key head in kf
        const bf16* kg = krow + ch;
#pragma unroll
        for (int h = 0; h < HP; ++h) {
            if (h < H) {
                if (left == 0) {
                    kf = make_uint4(0, 0, 0, 0);
                    if (key_ok && ch_ok) kf = *(const uint4*)kg;
                    kg += dim;
                    left = per;
                }
                --left;
                uint4 qa = make_uint4(0, 0, 0, 0), qb = qa;
                if (ch_ok) {
                    qa = *(const uint4*)(qa_row + (size_t)h * dim + c * 32);
                    qb = *(const uint4*)(qb_row + (size_t)h * dim + c * 32);
                }
                const uint32_t a1[4] = {qa.x, qb.x, qa.y, qb.y}, a2[4] = {qa.z, qb.z, qa.w, qb.w};
                mma_bf16(acc[h], a1, kf.x, kf.y);
                mma_bf16(acc[h], a2, kf.z, kf.w);
            }
        }
    }
    // accumulator places: (row gid, keys 2 t4 and 2 t4 + 1), (row gid + 8, the same keys)
    const int col = warp * 8 + 2 * t4;
    const float d0 = (float)(pos0 + gid - (b * PB + col));          // row gid's distance to its first key; row gid + 8: d0 + 8
#pragma unroll
    for (int h = 0; h < HP; ++h) {
        const float s = sl[h];
        acc[h][0] = acc[h][0] * p.scale - s * d0;
        acc[h][1] = acc[h][1] * p.scale - s * (d0 - 1.0f);
        acc[h][2] = acc[h][2] * p.scale - s * (d0 + 8.0f);
        acc[h][3] = acc[h][3] * p.scale - s * (d0 + 7.0f);
    }
    float* dst[2];
    bool live[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = gid + 8 * half, pos = pos0 + r;
        const int first = p.window > 0 ? max(0, pos - p.window + 1) / PB : 0;
        live[half] = r < n_rows && b >= first && b <= pos / PB;     // else the row sees nothing of this block
        dst[half] = p.mixed + (size_t)(row0 + r) * H * p.stride + (ptrdiff_t)(b - first) * PB + col;
    }
    const bool mix = p.talk.p != nullptr;
#pragma unroll
    for (int h = 0; h < HP; ++h) {
        if (h < H) {
            float m[4] = {acc[h][0], acc[h][1], acc[h][2], acc[h][3]};
            if (mix) {
                m[0] = m[1] = m[2] = m[3] = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < HP; g4 += 4) {
                    const float4 w = *(const float4*)(tk + h * HP + g4);
                    const float wa[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) m[e] = fmaf(wa[a], acc[g4 + a][e], m[e]);
                    }
                }
            }
            if (live[0]) *(float2*)(dst[0] + (size_t)h * p.stride) = make_float2(m[0], m[1]);
            if (live[1]) *(float2*)(dst[1] + (size_t)h * p.stride) = make_float2(m[2], m[3]);
        }
    }
}

__device__ __forceinline__ void ldsm4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// 64 rows of a sequence and one head: the softmax of the mixed scores, block of keys by block of keys with a running
// maximum and sum, and the weights times the values on the tensor cores.  A thread reads the scores of its places of the
// accumulator layout straight from memory (8-byte pairs), a block ahead of their use; the values of the next block arrive
// by cp.async in the other of two buffers meanwhile, as they lie in the cache ([key][channel]); ldmatrix.trans makes the
// B fragments of them.
template <int DV>
__global__ void __launch_bounds__(128, 3) talk_prompt_values_kernel(PromptArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int BM = 64, LV = DV + 8;
    bf16* sv = (bf16*)smem_raw;                                     // [2][PB][LV]
    const int seq = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
    const int qlen = p.seq_qlen[seq];
    if (q0 >= qlen) return;
    const int H = p.heads, G = p.kv_heads, vd = p.vdim;
    const int kvh = h / (H / G);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n_rows = min(BM, qlen - q0);
    fr_pdl_wait();
    fr_pdl_launch();
    const int row0 = p.seq_start[seq] + q0, pos0 = p.seq_pos0[seq] + q0, last_pos = pos0 + n_rows - 1;
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    int my_pos[2], my_first[2];
    const float* my_s[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        my_pos[half] = r < n_rows ? pos0 + r : -1;                  // a row beyond the sequence's sees nothing
        my_first[half] = p.window > 0 ? max(0, pos0 + r - p.window + 1) : 0;
        my_s[half] = p.mixed + ((size_t)(row0 + min(r, n_rows - 1)) * H + h) * p.stride + 2 * t;
    }
    // what the warp's 16 rows see, in blocks: others are skipped by the whole warp
    const int w_lo = (p.window > 0 ? max(0, pos0 + warp * 16 - p.window + 1) : 0) / PB;
    const int w_hi = min(pos0 + warp * 16 + 15, last_pos) / PB;
    const bool w_any = warp * 16 < n_rows;
    const int lo0 = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int b_lo = lo0 / PB, b_hi = last_pos / PB;
    const int* table = p.table + (size_t)seq * p.table_width;

    auto stage = [&](int b, int buf) {
        const bf16* vp = p.v_pool + ((size_t)table[b] * PB * G + kvh) * vd;
        bf16* dst = sv + (size_t)buf * PB * LV;
        for (int idx = tid; idx < PB * (DV / 8); idx += 128) {
            const int r = idx / (DV / 8), c = (idx - r * (DV / 8)) * 8;
            const bool ok = b * PB + r <= last_pos && c < vd;
            cp_async16(dst + r * LV + c, ok ? (const void*)(vp + (size_t)r * G * vd + c) : (const void*)p.v_pool, ok ? 16 : 0);
        }
        cp_commit();
    };
    // the scores of block b as they lie in memory: loads only, nothing depends on them until `finish` (a block later)
    auto fetch = [&](int b, float2 (&raw)[PB / 8][2]) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int pos = my_pos[half], first = my_first[half];
            const bool any = pos >= 0 && b >= first / PB && b <= pos / PB;
            const float* src = my_s[half] + (ptrdiff_t)(b - first / PB) * PB;
#pragma unroll
            for (int nt = 0; nt < PB / 8; ++nt) {
                raw[nt][half] = make_float2(-INFINITY, -INFINITY);
                if (any) raw[nt][half] = *(const float2*)(src + nt * 8);
            }
        }
    };
    // masked by position and scaled for a softmax on powers of two
    auto finish = [&](int b, const float2 (&raw)[PB / 8][2], float (&s)[PB / 8][4]) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int pos = my_pos[half], first = my_first[half];
            const bool whole = b * PB >= first && b * PB + PB - 1 <= pos;          // the row sees every key of the block
#pragma unroll
            for (int nt = 0; nt < PB / 8; ++nt) {
                float2 v = raw[nt][half];
                if (!whole) {
                    const int j = b * PB + nt * 8 + 2 * t;
                    if (j > pos || j < first) v.x = -INFINITY;
                    if (j + 1 > pos || j + 1 < first) v.y = -INFINITY;
                }
                s[nt][2 * half] = v.x * LOG2E;
                s[nt][2 * half + 1] = v.y * LOG2E;
            }
        }
    };

    float s[PB / 8][4];
    float2 raw[PB / 8][2];
    stage(b_lo, 0);
    fetch(b_lo, raw);
    finish(b_lo, raw, s);
    for (int b = b_lo; b <= b_hi; ++b) {
        const int buf = (b - b_lo) & 1;
        const bool more = b < b_hi;
        if (more) {
            stage(b + 1, buf ^ 1);
            fetch(b + 1, raw);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        if (w_any && b >= w_lo && b <= w_hi) {
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int nt = 0; nt < PB / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
            float corr[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 1));
                m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 2));
                corr[half] = m_new[half] == -INFINITY ? 1.f : exp2f(m_run[half] - m_new[half]);
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
#pragma unroll
            for (int nt = 0; nt < PB / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const float w = m_new[half] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_new[half]);
                    s[nt][e] = w;
                    l_run[half] += w;
                }
            }
            const bf16* vb = sv + (size_t)buf * PB * LV + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * LV + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < PB / 16; ++kk) {
                uint32_t hi[4], lw[4];
                split_bf16(s[2 * kk][0], s[2 * kk][1], hi[0], lw[0]);
                split_bf16(s[2 * kk][2], s[2 * kk][3], hi[1], lw[1]);
                split_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lw[2]);
                split_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lw[3]);
#pragma unroll
                for (int n2 = 0; n2 < DV / 16; ++n2) {
                    uint32_t vf[4];                                  // (keys 0-7, 8-15) x (channels n2 * 16, + 8)
                    ldsm4_trans(vf, vb + (size_t)kk * 16 * LV + n2 * 16);
                    mma_bf16(o[2 * n2], hi, vf[0], vf[1]);
                    mma_bf16(o[2 * n2 + 1], hi, vf[2], vf[3]);
                    mma_bf16(o[2 * n2], lw, vf[0], vf[1]);
                    mma_bf16(o[2 * n2 + 1], lw, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();                                            // the buffer is free for the block after next
        if (more) finish(b + 1, raw, s);
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
        const float inv = l_run[half] > 0.f ? 1.0f / l_run[half] : 0.f;
        bf16* dst = p.out + (size_t)(row0 + r) * H * vd + (size_t)h * vd;
        const bf16* gate = p.gate != nullptr ? p.gate + (size_t)(row0 + r) * p.gate_ld + (size_t)h * vd : nullptr;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int c = nt * 8 + 2 * t;
            if (c >= vd) continue;                                   // vd is even: c + 1 < vd as well
            float x = o[nt][2 * half] * inv, y = o[nt][2 * half + 1] * inv;
            if (gate != nullptr) {
                const __nv_bfloat162 gv = *(const __nv_bfloat162*)(gate + c);
                x *= 1.0f / (1.0f + expf(-__low2float(gv)));
                y *= 1.0f / (1.0f + expf(-__high2float(gv)));
            }
            *(uint32_t*)(dst + c) = pack_bf16(x, y);
        }
    }
}

template <int DV>
int launch_values(const PromptArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    const size_t smem = (size_t)2 * PB * (DV + 8) * sizeof(bf16);
    FR_CUDA(cudaFuncSetAttribute(talk_prompt_values_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((unsigned)((max_q_len + 63) / 64), (unsigned)p.heads, (unsigned)n_seqs);
    FR_CUDA(fr_launch(talk_prompt_values_kernel<DV>, grid, dim3(128), smem, stream, p));
    FR_CHECK_LAUNCH("talk prompt values");
    return FR_OK;
}

// elements per staged query row: all heads' channels and a pad that sets neighbouring rows 64 bytes apart modulo 128, so
// that the eight 16-byte reads of a quarter warp (two rows, four pieces each) meet no bank twice
int staged_row(int heads, int dim) {
    const int n = heads * dim;
    return n + ((32 - n % 64) + 64) % 64;
}

int padded_heads(int heads) { return heads <= 8 ? 8 : heads <= 16 ? 16 : heads <= 32 ? 32 : 0; }

size_t prompt_scores_smem(int heads, int dim) {
    const int hp = padded_heads(heads);
    return ((size_t)hp * hp + hp) * sizeof(float) + (size_t)QR * staged_row(heads, dim) * sizeof(bf16);
}

template <int HP>
int launch_scores(const PromptArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    const size_t smem = prompt_scores_smem(p.heads, p.dim);
    FR_CUDA(cudaFuncSetAttribute(talk_prompt_scores_kernel<HP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // a tile of 16 rows sees at most one block more than a single row does
    const dim3 grid((unsigned)(p.stride / PB + 1), (unsigned)((max_q_len + QR - 1) / QR), (unsigned)n_seqs);
    FR_CUDA(fr_launch(talk_prompt_scores_kernel<HP>, grid, dim3(256), smem, stream, p));
    FR_CHECK_LAUNCH("talk prompt scores");
    return FR_OK;
}

}  // namespace

// Floats of scratch memory for the mixed scores of n_rows rows; 0 if the tensor-core kernels do not take these sizes
// (key channels in eights, value channels in eights up to 128, what the score kernel holds in shared memory).
FR_EXPORT long long attention_talk_prompt_scratch_floats(int n_rows, int heads, int dim, int vdim, int window, int max_kv_len) {
    if (heads <= 0 || padded_heads(heads) == 0 || dim <= 0 || dim % 8 || vdim <= 0 || vdim % 8 || vdim > 128) return 0;
    if (prompt_scores_smem(heads, dim) > 200 * 1024) return 0;
    return (long long)n_rows * heads * prompt_stride(window, max_kv_len);
}

// bf16; pages of 64.  Sequences bring seq_qlen rows from row seq_start, the first at position seq_pos0; their keys and values
// are in the cache already.  q: [n_rows][q_ld], head h at h * dim; gate (or null): [n_rows][gate_ld]; out [n_rows][heads * vdim].
FR_EXPORT int attention_talk_prompt(const void* q, int q_ld, const void* k_pool, const void* v_pool, const int* table, int table_width,
                                    int page, const int* seq_start, const int* seq_qlen, const int* seq_pos0, int n_seqs, int n_rows,
                                    int max_q_len, int heads, int kv_heads, int dim, int vdim, int window, int max_kv_len, float scale,
                                    const float* slopes, const void* talk, int talk_dtype, const void* gate, int gate_ld, void* out,
                                    float* scratch, cudaStream_t stream) {
    if (n_seqs <= 0 || n_rows <= 0 || max_q_len <= 0) return FR_OK;
    if (page != PB) FR_REFUSE("talk prompt: pages of %d (64)", page);
    if (kv_heads <= 0 || heads % kv_heads) FR_REFUSE("talk prompt: %d heads cannot share %d key/value heads", heads, kv_heads);
    if (attention_talk_prompt_scratch_floats(n_rows, heads, dim, vdim, window, max_kv_len) <= 0)
        FR_REFUSE("talk prompt: %d heads of %d and %d are not sizes the tensor-core kernels take", heads, dim, vdim);
    if (n_seqs > 65535) FR_REFUSE("talk prompt: %d sequences", n_seqs);
    if ((uintptr_t)q % 16 || q_ld % 8 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (gate != nullptr && ((uintptr_t)gate % 4 || gate_ld % 2)))
        FR_REFUSE("talk prompt: rows and pools must start at 16 bytes");
    PromptArgs p;
    p.q = (const bf16*)q; p.q_ld = q_ld; p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool; p.table = table;
    p.table_width = table_width; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_pos0 = seq_pos0; p.heads = heads;
    p.kv_heads = kv_heads; p.dim = dim; p.q_ld_s = staged_row(heads, dim); p.vdim = vdim; p.window = window;
    p.stride = prompt_stride(window, max_kv_len); p.scale = scale; p.slopes = slopes; p.talk = FrVec{talk, talk_dtype};
    p.gate = (const bf16*)gate; p.gate_ld = gate_ld; p.out = (bf16*)out; p.mixed = scratch;
    const int hp = padded_heads(heads);
    const int rc = hp == 8 ? launch_scores<8>(p, n_seqs, max_q_len, stream)
                 : hp == 16 ? launch_scores<16>(p, n_seqs, max_q_len, stream) : launch_scores<32>(p, n_seqs, max_q_len, stream);
    if (rc != FR_OK) return rc;
    if (vdim <= 32) return launch_values<32>(p, n_seqs, max_q_len, stream);
    if (vdim <= 64) return launch_values<64>(p, n_seqs, max_q_len, stream);
    return launch_values<128>(p, n_seqs, max_q_len, stream);
}
