// Row-wise kernels for models whose residual stream is kept in 32-bit floats while their
// products run in the activation dtype: a norm that reads one dtype and writes another (with
// weights stored around zero or around one), [a; b] side by side in the activation dtype, the
// sum residual + alpha * y, the store of keys and values whose sizes differ, and the
// per-layer token input (a gated, normed projection of a small per-token table).
//
// All arithmetic is fp32; rounding happens only where a result is stored in bf16.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* residual_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

__device__ __forceinline__ float block_sum(float v, float* partial) {
    v = fr_warp_sum(v);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
    const int warps = (blockDim.x + 31) >> 5;
    for (int i = 0; i < warps; ++i) total += partial[i];
    __syncthreads();
    return total;
}

// y = x / sqrt(mean(x^2) + eps) * (offset + w), one block per row; x and y may differ in dtype.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
norm_cast_kernel(const TI* __restrict__ x, FrVec w, float offset, TO* __restrict__ y, int width, float eps) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const TI* xr = x + (size_t)blockIdx.x * width;
    TO* yr = y + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = fr_load(xr + i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) fr_store(yr + i, fr_load(xr + i) * inv * (offset + w.at(i)));
}

// out[r] = [a[r], b[r]] in the dtype of out
template <typename TI, typename TO>
__global__ void concat_cast_kernel(const TI* __restrict__ a, const TI* __restrict__ b, TO* __restrict__ out, int wa, int wb) {
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t r = blockIdx.x;
    TO* o = out + r * (size_t)(wa + wb);
    for (int i = threadIdx.x; i < wa; i += blockDim.x) fr_store(o + i, fr_load(a + r * wa + i));
    for (int i = threadIdx.x; i < wb; i += blockDim.x) fr_store(o + wa + i, fr_load(b + r * wb + i));
}

// out = residual + alpha * y (+ beta * z)
template <typename TY>
__global__ void add_scaled_kernel(const float* __restrict__ residual, const TY* __restrict__ y, float alpha,
                                  const TY* __restrict__ z, float beta, float* __restrict__ out, long long n) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = fmaf(alpha, fr_load(y + i), residual[i]);
        if (z != nullptr) v = fmaf(beta, fr_load(z + i), v);
        out[i] = v;
    }
}

// Keys [nkv][kd] at src + k_off and values [nkv][vd] at src + v_off of every live row go to the row of the paged
// cache that holds the row's position: pools [pages][page][nkv][kd] and [pages][page][nkv][vd].
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ src, int ld, int k_off, int v_off, int nkv, int kd, int vd,
                                const int* __restrict__ row_seq, const int* __restrict__ row_pos, T* __restrict__ k_pool,
                                T* __restrict__ v_pool, const int* __restrict__ block_table, int table_width, int page) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = row_pos[row];
    const int pg = block_table[(size_t)seq * table_width + pos / page];
    const size_t at = (size_t)pg * page + pos % page;
    const T* s = src + (size_t)row * ld;
    T* kd_ = k_pool + at * nkv * kd;
    T* vd_ = v_pool + at * nkv * vd;
    for (int i = threadIdx.x; i < nkv * kd; i += blockDim.x) kd_[i] = s[k_off + i];
    for (int i = threadIdx.x; i < nkv * vd; i += blockDim.x) vd_[i] = s[v_off + i];
}

// y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations, one block per row; two passes over
// the row, so that the variance is not a difference of large numbers.  x and y may differ in dtype.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
layernorm_cast_kernel(const TI* __restrict__ x, FrVec w, FrVec b, TO* __restrict__ y, int width, float eps) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const TI* xr = x + (size_t)blockIdx.x * width;
    TO* yr = y + (size_t)blockIdx.x * width;
    constexpr int KEEP = 16;                          // rows of up to 4,096 numbers are read once and kept in registers
    const bool kept = width <= KEEP * (int)blockDim.x;
    float v[KEEP];
    float sum = 0.f;
    if (kept) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            v[j] = i < width ? fr_load(xr + i) : 0.f;
            sum += v[j];
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) sum += fr_load(xr + i);
    }
    const float mean = block_sum(sum, partial) / (float)width;
    float ss = 0.f;
    if (kept) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            const float d = i < width ? v[j] - mean : 0.f;
            ss = fmaf(d, d, ss);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float d = fr_load(xr + i) - mean;
            ss = fmaf(d, d, ss);
        }
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    if (kept) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < width) {
                float o = (v[j] - mean) * inv * w.at(i);
                if (b.p != nullptr) o += b.at(i);
                fr_store(yr + i, o);
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float o = (fr_load(xr + i) - mean) * inv * w.at(i);
            if (b.p != nullptr) o += b.at(i);
            fr_store(yr + i, o);
        }
    }
}

// out[r] = table[tokens[r]] * scale as 32-bit rows (ids outside the table leave zeros)
template <typename TW>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, float* __restrict__ out, int width,
                                  int vocab, float scale) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int token = tokens[blockIdx.x];
    float* o = out + (size_t)blockIdx.x * width;
    const bool ok = token >= 0 && token < vocab;
    const TW* t = table + (size_t)(ok ? token : 0) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = ok ? fr_load(t + i) * scale : 0.f;
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The per-layer token input, in place on the 32-bit residual stream:
//   e = table[token][col0 .. col0 + dim);  g = gelu_tanh(gate x) * e;  y = proj g;
//   x += y / sqrt(mean(y^2) + eps) * norm
// gate [dim][width], proj [width][dim], norm [width], table [vocab][table_ld] in the dtype TW.  Two kernels: a warp per
// (row, channel of g), then a block per row for the projection, its norm and the sum.
template <typename TW>
__global__ void __launch_bounds__(128)
token_gate_kernel(const float* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ row_seq,
                  const TW* __restrict__ table, int table_ld, int col0, int vocab, const TW* __restrict__ gate,
                  float* __restrict__ g, int rows, int width, int dim) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= rows * dim) return;
    const int row = item / dim, d = item - row * dim;
    const int token = tokens[row];
    if ((row_seq != nullptr && row_seq[row] < 0) || token < 0 || token >= vocab) return;
    const float* xr = x + (size_t)row * width;
    const TW* gr = gate + (size_t)d * width;
    float s = 0.f;
    constexpr int PER = 16 / sizeof(TW);
    if (width % PER == 0 && ((((uintptr_t)xr) | ((uintptr_t)gr)) & 15) == 0) {
        for (int c = lane * PER; c < width; c += 32 * PER) {
            const uint4 wv = *(const uint4*)(gr + c);
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const float4 xv = *(const float4*)(xr + c + i);
                s = fmaf(xv.x, fr_load((const TW*)&wv + i), s);
                s = fmaf(xv.y, fr_load((const TW*)&wv + i + 1), s);
                s = fmaf(xv.z, fr_load((const TW*)&wv + i + 2), s);
                s = fmaf(xv.w, fr_load((const TW*)&wv + i + 3), s);
            }
        }
    } else {
        for (int c = lane; c < width; c += 32) s = fmaf(xr[c], fr_load(gr + c), s);
    }
    s = fr_warp_sum(s);
    if (lane == 0) g[(size_t)row * dim + d] = gelu_tanh(s) * fr_load(table + (size_t)token * table_ld + col0 + d);
}

template <typename TW>
__global__ void __launch_bounds__(1024)
token_proj_kernel(float* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ row_seq, int vocab,
                  const float* __restrict__ gs, const TW* __restrict__ proj, FrVec norm, int width, int dim, float eps) {
    extern __shared__ float sm[];
    float* g = sm;                // [dim]
    float* y = sm + dim;          // [width]
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int token = tokens[row];
    if ((row_seq != nullptr && row_seq[row] < 0) || token < 0 || token >= vocab) return;
    float* xr = x + (size_t)row * width;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) g[d] = gs[(size_t)row * dim + d];
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const TW* pr = proj + (size_t)c * dim;
        float s = 0.f;
        constexpr int PER = 16 / sizeof(TW);
        if (dim % PER == 0 && (((uintptr_t)pr) & 15) == 0) {
            for (int d = 0; d < dim; d += PER) {
                const uint4 pv = *(const uint4*)(pr + d);
#pragma unroll
                for (int i = 0; i < PER; ++i) s = fmaf(g[d + i], fr_load((const TW*)&pv + i), s);
            }
        } else {
            for (int d = 0; d < dim; ++d) s = fmaf(g[d], fr_load(pr + d), s);
        }
        y[c] = s;
        ss = fmaf(s, s, ss);
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) xr[c] += y[c] * inv * norm.at(c);
}

// Many rows: the two projections run as products; these are the steps between them.
// g[row][d] = gelu_tanh(z[row][d]) * table[token][col0 + d], in the dtype of g
template <typename TW>
__global__ void gelu_table_kernel(const float* __restrict__ z, const int* __restrict__ tokens, const TW* __restrict__ table,
                                  int table_ld, int col0, int vocab, TW* __restrict__ g, int rows, int dim) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < rows * dim; idx += gridDim.x * blockDim.x) {
        const int row = idx / dim, d = idx - row * dim;
        const int token = tokens[row];
        const float e = token >= 0 && token < vocab ? fr_load(table + (size_t)token * table_ld + col0 + d) : 0.f;
        fr_store(g + idx, gelu_tanh(z[idx]) * e);
    }
}

// x += y / sqrt(mean(y^2) + eps) * norm, one block per row
__global__ void __launch_bounds__(256) rms_add_kernel(float* __restrict__ x, const float* __restrict__ y, FrVec norm, int width, float eps) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    float* xr = x + (size_t)blockIdx.x * width;
    const float* yr = y + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) xr[c] += yr[c] * inv * norm.at(c);
}

inline int blocks_for(long long n) {
    const long long cap = (long long)(fr_sm_count() > 0 ? fr_sm_count() : 128) * 16;
    const long long want = (n + 255) / 256;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace

FR_EXPORT int residual_norm_cast(const void* x, int in_dtype, const void* w, int w_dtype, float offset, void* y, int out_dtype,
                                 int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FrVec wv{w, w_dtype};
    const int key = in_dtype * 2 + out_dtype;
    switch (key) {
        case 0: FR_CUDA(fr_launch(norm_cast_kernel<float, float>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, offset, (float*)y, width, eps)); break;
        case 1: FR_CUDA(fr_launch(norm_cast_kernel<float, bf16>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, offset, (bf16*)y, width, eps)); break;
        case 2: FR_CUDA(fr_launch(norm_cast_kernel<bf16, float>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, offset, (float*)y, width, eps)); break;
        case 3: FR_CUDA(fr_launch(norm_cast_kernel<bf16, bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, offset, (bf16*)y, width, eps)); break;
        default: FR_REFUSE("norm_cast: unknown dtypes %d -> %d", in_dtype, out_dtype);
    }
    FR_CHECK_LAUNCH("norm_cast");
    return FR_OK;
}

FR_EXPORT int residual_concat_cast(const void* a, const void* b, int in_dtype, void* out, int out_dtype, int n_rows, int wa,
                                   int wb, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const int key = in_dtype * 2 + out_dtype;
    switch (key) {
        case 0: FR_CUDA(fr_launch(concat_cast_kernel<float, float>, dim3(n_rows), dim3(256), 0, stream, (const float*)a, (const float*)b, (float*)out, wa, wb)); break;
        case 1: FR_CUDA(fr_launch(concat_cast_kernel<float, bf16>, dim3(n_rows), dim3(256), 0, stream, (const float*)a, (const float*)b, (bf16*)out, wa, wb)); break;
        case 2: FR_CUDA(fr_launch(concat_cast_kernel<bf16, float>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, (float*)out, wa, wb)); break;
        case 3: FR_CUDA(fr_launch(concat_cast_kernel<bf16, bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, (bf16*)out, wa, wb)); break;
        default: FR_REFUSE("concat_cast: unknown dtypes %d -> %d", in_dtype, out_dtype);
    }
    FR_CHECK_LAUNCH("concat_cast");
    return FR_OK;
}

// out [n] fp32 = residual [n] fp32 + alpha * y [n] (+ beta * z [n]); y and z in y_dtype; out may be residual.
FR_EXPORT int residual_add_scaled(const float* residual, const void* y, float alpha, const void* z, float beta, int y_dtype,
                                  float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    if (y_dtype == FR_F32)
        FR_CUDA(fr_launch(add_scaled_kernel<float>, dim3(blocks_for(n)), dim3(256), 0, stream, residual, (const float*)y, alpha,
                          (const float*)z, beta, out, n));
    else if (y_dtype == FR_BF16)
        FR_CUDA(fr_launch(add_scaled_kernel<bf16>, dim3(blocks_for(n)), dim3(256), 0, stream, residual, (const bf16*)y, alpha,
                          (const bf16*)z, beta, out, n));
    else
        FR_REFUSE("add_scaled: unknown dtype %d", y_dtype);
    FR_CHECK_LAUNCH("add_scaled");
    return FR_OK;
}

FR_EXPORT int residual_kv_store(const void* src, int ld, int k_off, int v_off, int nkv, int kd, int vd, const int* row_seq,
                                const int* row_pos, void* k_pool, void* v_pool, const int* block_table, int table_width,
                                int page, int n_rows, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (k_pool == nullptr || v_pool == nullptr || block_table == nullptr) FR_REFUSE("kv_store: no cache to write to");
    if (dtype == FR_F32)
        FR_CUDA(fr_launch(kv_store_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)src, ld, k_off, v_off, nkv, kd,
                          vd, row_seq, row_pos, (float*)k_pool, (float*)v_pool, block_table, table_width, page));
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(kv_store_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (const bf16*)src, ld, k_off, v_off, nkv, kd,
                          vd, row_seq, row_pos, (bf16*)k_pool, (bf16*)v_pool, block_table, table_width, page));
    else
        FR_REFUSE("kv_store: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("kv_store");
    return FR_OK;
}

// g_scratch: [n_rows][dim] floats
FR_EXPORT int residual_token_input(float* x, const int* tokens, const int* row_seq, const void* table, int table_ld, int col0,
                                   int vocab, const void* gate, const void* proj, const void* norm, int norm_dtype, int n_rows,
                                   int width, int dim, float eps, float* g_scratch, int w_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (g_scratch == nullptr) FR_REFUSE("token_input: no scratch for the gated table rows");
    const size_t smem = (size_t)(dim + width) * sizeof(float);
    if (smem > 200 * 1024) FR_REFUSE("token_input: width %d and dim %d need more shared memory than an SM has", width, dim);
    FrVec nv{norm, norm_dtype};
    const int gate_blocks = (int)(((long long)n_rows * dim + 3) / 4);
    const int threads = n_rows < 128 ? 1024 : 256;            // few rows: more threads each, to keep loads in flight
    if (w_dtype == FR_F32) {
        FR_CUDA(fr_launch(token_gate_kernel<float>, dim3(gate_blocks), dim3(128), 0, stream, (const float*)x, tokens, row_seq,
                          (const float*)table, table_ld, col0, vocab, (const float*)gate, g_scratch, n_rows, width, dim));
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(token_proj_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(token_proj_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, tokens, row_seq, vocab,
                          (const float*)g_scratch, (const float*)proj, nv, width, dim, eps));
    } else if (w_dtype == FR_BF16) {
        FR_CUDA(fr_launch(token_gate_kernel<bf16>, dim3(gate_blocks), dim3(128), 0, stream, (const float*)x, tokens, row_seq,
                          (const bf16*)table, table_ld, col0, vocab, (const bf16*)gate, g_scratch, n_rows, width, dim));
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(token_proj_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(token_proj_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, tokens, row_seq, vocab,
                          (const float*)g_scratch, (const bf16*)proj, nv, width, dim, eps));
    } else {
        FR_REFUSE("token_input: unknown dtype %d", w_dtype);
    }
    FR_CHECK_LAUNCH("token_input");
    return FR_OK;
}

FR_EXPORT int residual_gelu_table(const float* z, const int* tokens, const void* table, int table_ld, int col0, int vocab, void* g,
                                  int rows, int dim, int w_dtype, cudaStream_t stream) {
    if (rows <= 0 || dim <= 0) return FR_OK;
    const int blocks = blocks_for((long long)rows * dim);
    if (w_dtype == FR_F32) FR_CUDA(fr_launch(gelu_table_kernel<float>, dim3(blocks), dim3(256), 0, stream, z, tokens, (const float*)table, table_ld, col0, vocab, (float*)g, rows, dim));
    else if (w_dtype == FR_BF16) FR_CUDA(fr_launch(gelu_table_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, z, tokens, (const bf16*)table, table_ld, col0, vocab, (bf16*)g, rows, dim));
    else FR_REFUSE("gelu_table: unknown dtype %d", w_dtype);
    FR_CHECK_LAUNCH("gelu_table");
    return FR_OK;
}

FR_EXPORT int residual_rms_add(float* x, const float* y, const void* norm, int norm_dtype, int rows, int width, float eps, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    FR_CUDA(fr_launch(rms_add_kernel, dim3(rows), dim3(256), 0, stream, x, y, FrVec{norm, norm_dtype}, width, eps));
    FR_CHECK_LAUNCH("rms_add");
    return FR_OK;
}

// bias null: none.  The weight and the bias share a dtype.
FR_EXPORT int residual_layernorm_cast(const void* x, int in_dtype, const void* w, const void* b, int w_dtype, void* y, int out_dtype,
                                      int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FrVec wv{w, w_dtype}, bv{b, w_dtype};
    const int key = in_dtype * 2 + out_dtype;
    switch (key) {
        case 0: FR_CUDA(fr_launch(layernorm_cast_kernel<float, float>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, bv, (float*)y, width, eps)); break;
        case 1: FR_CUDA(fr_launch(layernorm_cast_kernel<float, bf16>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, bv, (bf16*)y, width, eps)); break;
        case 2: FR_CUDA(fr_launch(layernorm_cast_kernel<bf16, float>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, bv, (float*)y, width, eps)); break;
        case 3: FR_CUDA(fr_launch(layernorm_cast_kernel<bf16, bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, bv, (bf16*)y, width, eps)); break;
        default: FR_REFUSE("layernorm_cast: unknown dtypes %d -> %d", in_dtype, out_dtype);
    }
    FR_CHECK_LAUNCH("layernorm_cast");
    return FR_OK;
}

FR_EXPORT int residual_embed_rows(const int* tokens, const void* table, int table_dtype, float* out, int n_rows, int width, int vocab,
                                  float scale, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (table_dtype == FR_F32) FR_CUDA(fr_launch(embed_rows_kernel<float>, dim3(n_rows), dim3(256), 0, stream, tokens, (const float*)table, out, width, vocab, scale));
    else if (table_dtype == FR_BF16) FR_CUDA(fr_launch(embed_rows_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, tokens, (const bf16*)table, out, width, vocab, scale));
    else FR_REFUSE("embed_rows: unknown dtype %d", table_dtype);
    FR_CHECK_LAUNCH("embed_rows");
    return FR_OK;
}

// ------------------------------------------------------------------ a learned position table, token shift, norms around a sublayer
namespace {

// out[r] = table[token[r]] + positions[pos[r]], 32-bit
template <typename TW>
__global__ void embed_pos_kernel(const int* __restrict__ tokens, const int* __restrict__ row_pos, const TW* __restrict__ table,
                                 const TW* __restrict__ positions, float* __restrict__ out, int width, int vocab, int max_pos) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int token = tokens[blockIdx.x], pos = row_pos[blockIdx.x];
    float* o = out + (size_t)blockIdx.x * width;
    const bool ok = token >= 0 && token < vocab && pos >= 0 && pos < max_pos;
    const TW* t = table + (size_t)(ok ? token : 0) * width;
    const TW* q = positions + (size_t)(ok ? pos : 0) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = ok ? fr_load(t + i) + fr_load(q + i) : 0.f;
}

// h = x / sqrt(mean(x^2) + eps) * w per row; y = h + (h_before - h) * shift, where h_before is the same norm of the row
// before in the sequence, or the sequence's kept row (state) for the first row of a step.  save: every row also leaves its
// h in the state (steps of one row per sequence, where the block that reads the state is the one that writes it).
template <typename TO>
__global__ void __launch_bounds__(256)
norm_shift_kernel(const float* __restrict__ x, FrVec w, FrVec shift, TO* __restrict__ y, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ row_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slots, int width,
                  float eps, int save) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    if (seq < 0) return;
    const bool first = row == seq_start[seq];
    const float* xr = x + (size_t)row * width;
    const float* xb = xr - width;
    float* sp = state + (size_t)seq_slots[seq] * state_stride;
    float ss = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
        if (!first) {
            const float u = xb[i];
            sb = fmaf(u, u, sb);
        }
    }
    ss = block_sum(ss, partial);
    sb = block_sum(sb, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps), invb = 1.0f / sqrtf(sb / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float wi = w.at(i);
        const float h = xr[i] * inv * wi;
        const float before = first ? sp[i] : xb[i] * invb * wi;
        fr_store(y + (size_t)row * width + i, fmaf(before - h, shift.at(i), h));
        if (save) sp[i] = h;
    }
}

// the state keeps the norm of every sequence's last row of the step
__global__ void __launch_bounds__(256)
norm_keep_last_kernel(const float* __restrict__ x, FrVec w, float* __restrict__ state, long long state_stride,
                      const int* __restrict__ seq_start, const int* __restrict__ seq_qlen, const int* __restrict__ seq_slots, int width,
                      float eps) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const int seq = blockIdx.x;
    const int n = seq_qlen[seq];
    if (n <= 0) return;
    const float* xr = x + (size_t)(seq_start[seq] + n - 1) * width;
    float* sp = state + (size_t)seq_slots[seq] * state_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) sp[i] = xr[i] * inv * w.at(i);
}

// out = x + mult * y / sqrt(mean(y^2) + eps) * w; and, if asked for, the norm of `out` that the next sublayer reads:
// next = out / sqrt(mean(out^2) + eps2) * w2 in the activation dtype
template <typename TO>
__global__ void __launch_bounds__(256)
post_norm_add_kernel(const float* __restrict__ x, const float* __restrict__ y, FrVec w, float eps, float mult, float* __restrict__ out,
                     FrVec w2, float eps2, TO* __restrict__ next, int width) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(y[base + i], y[base + i], ss);
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float o = fmaf(mult, y[base + i] * inv * w.at(i), x[base + i]);
        out[base + i] = o;
        s2 = fmaf(o, o, s2);
    }
    if (next == nullptr) return;
    s2 = block_sum(s2, partial);
    const float inv2 = 1.0f / sqrtf(s2 / (float)width + eps2);
    for (int i = threadIdx.x; i < width; i += blockDim.x) fr_store(next + base + i, out[base + i] * inv2 * w2.at(i));
}

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2;  (p, q) = pq[0], pq[1]
template <typename T>
__global__ void two_sided_act_kernel(T* __restrict__ z, long long n, FrVec pq) {
    fr_pdl_wait();
    fr_pdl_launch();
    const float a = softplus_f(pq.at(0)), b = 0.5f + softplus_f(pq.at(1));
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fr_load(z + i);
        fr_store(z + i, v > 0.f ? fmaf(a * v, v, 0.5f * v) : fmaf(b, expm1f(v) - v, 0.5f * v));
    }
}

// ---- the same three row-wise kernels for rows of whole 16-byte pieces that a block can hold in registers (a thread keeps
// NV pieces of four floats): every input is read once, 16 bytes at a time, and the arithmetic is the scalar kernels'.
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *(uint2*)p = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
}

template <typename TO, int NV>
__global__ void __launch_bounds__(256)
norm_shift_vec_kernel(const float* __restrict__ x, FrVec w, FrVec shift, TO* __restrict__ y, float* __restrict__ state, long long state_stride,
                      const int* __restrict__ row_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slots, int width,
                      float eps, int save) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    if (seq < 0) return;
    const bool first = row == seq_start[seq];
    const float4* xr = (const float4*)(x + (size_t)row * width);
    const float4* xb = (const float4*)(x + (size_t)row * width - width);
    float* sp = state + (size_t)seq_slots[seq] * state_stride;
    const int n4 = width >> 2;
    float4 a[NV], b[NV];
    float ss = 0.f, sb = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            a[k] = xr[i];
            b[k] = first ? ((const float4*)sp)[i] : xb[i];
        }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            ss = fmaf(a[k].x, a[k].x, ss); ss = fmaf(a[k].y, a[k].y, ss); ss = fmaf(a[k].z, a[k].z, ss); ss = fmaf(a[k].w, a[k].w, ss);
            if (!first) {
                sb = fmaf(b[k].x, b[k].x, sb); sb = fmaf(b[k].y, b[k].y, sb); sb = fmaf(b[k].z, b[k].z, sb); sb = fmaf(b[k].w, b[k].w, sb);
            }
        }
    }
    ss = block_sum(ss, partial);
    sb = block_sum(sb, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps), invb = 1.0f / sqrtf(sb / (float)width + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float av[4] = {a[k].x, a[k].y, a[k].z, a[k].w}, bv[4] = {b[k].x, b[k].y, b[k].z, b[k].w};
            float h[4], o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float wi = w.at(4 * i + e);
                h[e] = av[e] * inv * wi;
                const float before = first ? bv[e] : bv[e] * invb * wi;
                o[e] = fmaf(before - h[e], shift.at(4 * i + e), h[e]);
            }
            store4(y + (size_t)row * width + 4 * i, o);
            if (save) store4(sp + 4 * i, h);
        }
    }
}

template <typename TO, int NV>
__global__ void __launch_bounds__(256)
post_norm_add_vec_kernel(const float* __restrict__ x, const float* __restrict__ y, FrVec w, float eps, float mult, float* __restrict__ out,
                         FrVec w2, float eps2, TO* __restrict__ next, int width) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t base = (size_t)blockIdx.x * width;
    const int n4 = width >> 2;
    float4 v[NV], r[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            v[k] = ((const float4*)(y + base))[i];
            r[k] = ((const float4*)(x + base))[i];
        }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) { ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss); }
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float yv[4] = {v[k].x, v[k].y, v[k].z, v[k].w}, xv[4] = {r[k].x, r[k].y, r[k].z, r[k].w};
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[e] = fmaf(mult, yv[e] * inv * w.at(4 * i + e), xv[e]);
                s2 = fmaf(o[e], o[e], s2);
            }
            store4(out + base + 4 * i, o);
            v[k] = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
    if (next == nullptr) return;
    s2 = block_sum(s2, partial);
    const float inv2 = 1.0f / sqrtf(s2 / (float)width + eps2);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float ov[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = ov[e] * inv2 * w2.at(4 * i + e);
            store4(next + base + 4 * i, o);
        }
    }
}

// 16 bytes of z per thread and turn
template <typename T>
__global__ void two_sided_act_vec_kernel(T* __restrict__ z, long long pieces, FrVec pq) {
    constexpr int PER = 16 / (int)sizeof(T);
    fr_pdl_wait();
    fr_pdl_launch();
    const float a = softplus_f(pq.at(0)), b = 0.5f + softplus_f(pq.at(1));
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (long long)gridDim.x * blockDim.x) {
        uint4 raw = ((const uint4*)z)[i];
        T* e = (T*)&raw;
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const float v = fr_load(e + k);
            fr_store(e + k, v > 0.f ? fmaf(a * v, v, 0.5f * v) : fmaf(b, expm1f(v) - v, 0.5f * v));
        }
        ((uint4*)z)[i] = raw;
    }
}

}  // namespace

FR_EXPORT int residual_embed_pos(const int* tokens, const int* row_pos, const void* table, const void* positions, int table_dtype, float* out,
                                 int n_rows, int width, int vocab, int max_pos, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (table_dtype == FR_F32)
        FR_CUDA(fr_launch(embed_pos_kernel<float>, dim3(n_rows), dim3(256), 0, stream, tokens, row_pos, (const float*)table,
                          (const float*)positions, out, width, vocab, max_pos));
    else if (table_dtype == FR_BF16)
        FR_CUDA(fr_launch(embed_pos_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, tokens, row_pos, (const bf16*)table,
                          (const bf16*)positions, out, width, vocab, max_pos));
    else FR_REFUSE("embed_pos: unknown dtype %d", table_dtype);
    FR_CHECK_LAUNCH("embed_pos");
    return FR_OK;
}

// decode != 0: every sequence brings one row (the rows keep their norms themselves); otherwise a second kernel keeps the
// norm of every sequence's last row once all rows have read what the state held.
FR_EXPORT int residual_norm_shift(const float* x, const void* w, int w_dtype, const void* shift, int shift_dtype, void* y, int out_dtype,
                                  float* state, long long state_stride, const int* row_seq, const int* seq_start, const int* seq_qlen,
                                  const int* seq_slots, int n_rows, int n_seqs, int width, float eps, int decode, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (state == nullptr || state_stride < width) FR_REFUSE("norm_shift: a state of at least the width per sequence");
    const FrVec wv{w, w_dtype}, sv{shift, shift_dtype};
    const bool pieces = width % 4 == 0 && width <= 8192 && state_stride % 4 == 0 &&
                        ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)state)) & 15) == 0;
#define SHIFT_VEC(TO, NV)                                                                                                          \
    FR_CUDA(fr_launch(norm_shift_vec_kernel<TO, NV>, dim3(n_rows), dim3(256), 0, stream, x, wv, sv, (TO*)y, state, state_stride, row_seq, \
                      seq_start, seq_slots, width, eps, decode ? 1 : 0))
    if (pieces && out_dtype == FR_F32) {
        if (width <= 2048) SHIFT_VEC(float, 2); else if (width <= 4096) SHIFT_VEC(float, 4); else SHIFT_VEC(float, 8);
    } else if (pieces && out_dtype == FR_BF16) {
        if (width <= 2048) SHIFT_VEC(bf16, 2); else if (width <= 4096) SHIFT_VEC(bf16, 4); else SHIFT_VEC(bf16, 8);
    } else if (out_dtype == FR_F32)
#undef SHIFT_VEC
        FR_CUDA(fr_launch(norm_shift_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, wv, sv, (float*)y, state, state_stride, row_seq,
                          seq_start, seq_slots, width, eps, decode ? 1 : 0));
    else if (out_dtype == FR_BF16)
        FR_CUDA(fr_launch(norm_shift_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, x, wv, sv, (bf16*)y, state, state_stride, row_seq,
                          seq_start, seq_slots, width, eps, decode ? 1 : 0));
    else FR_REFUSE("norm_shift: unknown dtype %d", out_dtype);
    FR_CHECK_LAUNCH("norm_shift");
    if (!decode) {
        FR_CUDA(fr_launch(norm_keep_last_kernel, dim3(n_seqs), dim3(256), 0, stream, x, wv, state, state_stride, seq_start, seq_qlen,
                          seq_slots, width, eps));
        FR_CHECK_LAUNCH("norm_keep_last");
    }
    return FR_OK;
}

FR_EXPORT int residual_post_norm_add(const float* x, const float* y, const void* w, int w_dtype, float eps, float mult, float* out,
                                     const void* w2, int w2_dtype, float eps2, void* next, int next_dtype, int n_rows, int width,
                                     cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const FrVec wv{w, w_dtype}, w2v{w2, w2_dtype};
    const bool pieces = width % 4 == 0 && width <= 8192 &&
                        ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)out) | ((uintptr_t)next)) & 15) == 0;
#define POST_VEC(TO, NV)                                                                                                           \
    FR_CUDA(fr_launch(post_norm_add_vec_kernel<TO, NV>, dim3(n_rows), dim3(256), 0, stream, x, y, wv, eps, mult, out, w2v, eps2, (TO*)next, width))
    if (pieces && (next == nullptr || next_dtype == FR_F32)) {
        if (width <= 2048) POST_VEC(float, 2); else if (width <= 4096) POST_VEC(float, 4); else POST_VEC(float, 8);
    } else if (pieces && next_dtype == FR_BF16) {
        if (width <= 2048) POST_VEC(bf16, 2); else if (width <= 4096) POST_VEC(bf16, 4); else POST_VEC(bf16, 8);
    } else if (next == nullptr || next_dtype == FR_F32)
#undef POST_VEC
        FR_CUDA(fr_launch(post_norm_add_kernel<float>, dim3(n_rows), dim3(256), 0, stream, x, y, wv, eps, mult, out, w2v, eps2, (float*)next, width));
    else if (next_dtype == FR_BF16)
        FR_CUDA(fr_launch(post_norm_add_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, x, y, wv, eps, mult, out, w2v, eps2, (bf16*)next, width));
    else FR_REFUSE("post_norm_add: unknown dtype %d", next_dtype);
    FR_CHECK_LAUNCH("post_norm_add");
    return FR_OK;
}

FR_EXPORT int residual_two_sided_act(void* z, long long n, int dtype, const void* pq, int pq_dtype, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    const FrVec v{pq, pq_dtype};
    const long long per = dtype == FR_F32 ? 4 : 8;
    if ((dtype == FR_F32 || dtype == FR_BF16) && n % per == 0 && ((uintptr_t)z & 15) == 0) {
        const long long pieces = n / per;
        const unsigned vb = (unsigned)((pieces + 255) / 256 < 148 * 16 ? (pieces + 255) / 256 : 148 * 16);
        if (dtype == FR_F32) FR_CUDA(fr_launch(two_sided_act_vec_kernel<float>, dim3(vb), dim3(256), 0, stream, (float*)z, pieces, v));
        else FR_CUDA(fr_launch(two_sided_act_vec_kernel<bf16>, dim3(vb), dim3(256), 0, stream, (bf16*)z, pieces, v));
        FR_CHECK_LAUNCH("two_sided_act");
        return FR_OK;
    }
    const unsigned blocks = (unsigned)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    if (dtype == FR_F32) FR_CUDA(fr_launch(two_sided_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)z, n, v));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(two_sided_act_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)z, n, v));
    else FR_REFUSE("two_sided_act: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("two_sided_act");
    return FR_OK;
}

// ------------------------------------------------------------------ a hashed token-pair table beside the token table
// out[row] = table[token] + pairs[r] as 32-bit rows, r = (previous token * mul_prev + token * mul_cur) mod buckets, or row
// `buckets` (the table's last) for a sequence's first token.  The previous token of a step's first row comes from the
// sequence's state (one int32 per slot), which then keeps the step's last token: the block of a sequence's first row reads
// the state before it writes it, and no other block touches it.
namespace {

template <typename TW>
__global__ void __launch_bounds__(256)
embed_pair_kernel(const int* __restrict__ tokens, const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                  const int* __restrict__ seq_start, const int* __restrict__ seq_qlen, const int* __restrict__ seq_slots,
                  const TW* __restrict__ table, const TW* __restrict__ pairs, int* __restrict__ state, float* __restrict__ out, int width,
                  int vocab, int buckets, long long mul_prev, long long mul_cur) {
    fr_pdl_wait();
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    float* o = out + (size_t)row * width;
    if (seq < 0) {
        fr_pdl_launch();
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const int token = tokens[row], pos = row_pos[row], first = seq_start[seq];
    int prev = 0;
    if (pos > 0) prev = row > first ? tokens[row - 1] : state[seq_slots[seq]];
    __syncthreads();                                  // every thread has read the state before one of them writes it
    if (row == first && threadIdx.x == 0) state[seq_slots[seq]] = tokens[first + seq_qlen[seq] - 1];
    fr_pdl_launch();
    const bool ok = token >= 0 && token < vocab;
    const long long r = pos > 0 ? ((long long)prev * mul_prev + (long long)token * mul_cur) % (long long)buckets : (long long)buckets;
    const TW* t = table + (size_t)(ok ? token : 0) * width;
    const TW* b = pairs + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = ok ? fr_load(t + i) + fr_load(b + i) : 0.f;
}

// ------------------------------------------------------------------ layer norm, then a short causal convolution added to it
// h = layer_norm(x) rounded to the result's dtype; y_t = h_t + sum_j taps[:, j] * h_(t - n + 1 + j) (n taps; rows before the
// sequence's start are zero).  Rows before a step's first come from the sequence's state: its last n - 1 rows h, oldest
// first, 32-bit.  One block per row; the block norms the n - 1 rows before its own again instead of reading them from
// memory that another block would have to write first.
template <typename TO> __device__ __forceinline__ float round_as(float v);
template <> __device__ __forceinline__ float round_as<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_as<bf16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct NormConvArgs {
    const float* x;          // [rows][width]
    FrVec w, b, taps;        // layer norm's weight and bias (b.p null: none); taps [width][n]
    void* y;                 // [rows][width]
    float* state;            // [slots][stride]: (n - 1) rows of width numbers at `offset`
    long long stride, offset;
    const int* row_seq;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_slots;
    int width, n, shift;     // shift: every sequence brings one row and the history moves on in the same kernel
    int rows, tile, cols;    // rows of the step; rows per block; columns per block
    float eps;
};

constexpr int CONV_MAX_TAPS = 8, CONV_TILE = 4;

// mean and 1 / sqrt(variance + eps) of one row, by one warp (the variance is the mean of the squared deviations).  Rows of up
// to 2,048 numbers in whole 16-byte pieces are read once, every load issued before any is used, and kept in registers for the
// second sum; others are read twice.
__device__ __forceinline__ void warp_row_stats(const float* xr, int width, float eps, int lane, float& mean, float& inv) {
    constexpr int KEEP = 16;
    float sum = 0.f, ss = 0.f;
    const bool pieces = (width & 3) == 0 && (((uintptr_t)xr) & 15) == 0;
    if (pieces && width <= KEEP * 128) {
        const float4* x4 = (const float4*)xr;
        float4 v[KEEP];
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = lane + 32 * j;
            v[j] = i < width / 4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < KEEP; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        mean = fr_warp_sum(sum) / (float)width;
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            if (lane + 32 * j < width / 4) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                ss += (a * a + b * b) + (c * c + d * d);
            }
        }
    } else if (pieces) {
        const float4* x4 = (const float4*)xr;
#pragma unroll 8
        for (int i = lane; i < width / 4; i += 32) {
            const float4 v = x4[i];
            sum += (v.x + v.y) + (v.z + v.w);
        }
        mean = fr_warp_sum(sum) / (float)width;
#pragma unroll 8
        for (int i = lane; i < width / 4; i += 32) {
            const float4 v = x4[i];
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            ss += (a * a + b * b) + (c * c + d * d);
        }
    } else {
        for (int i = lane; i < width; i += 32) sum += xr[i];
        mean = fr_warp_sum(sum) / (float)width;
        for (int i = lane; i < width; i += 32) {
            const float d = xr[i] - mean;
            ss = fmaf(d, d, ss);
        }
    }
    inv = 1.0f / sqrtf(fr_warp_sum(ss) / (float)width + eps);
}

// A block owns `tile` consecutive rows of the step and `cols` columns.  Its warps first take the statistics of those rows and
// of the n - 1 rows before them (once per row, not once per tap), then every thread walks its columns: the normed rows that
// the taps reach are formed again from x (they are in L1 by then) or, before a step's first row, read from the history.
template <typename TO>
__global__ void __launch_bounds__(256) norm_conv_kernel(NormConvArgs p) {
    __shared__ float stats[CONV_TILE + CONV_MAX_TAPS][2];
    fr_pdl_wait();
    fr_pdl_launch();
    const int r0 = blockIdx.x * p.tile, r1 = min(r0 + p.tile, p.rows);
    const int first = p.shift ? r0 : max(0, r0 - (p.n - 1));          // one row per sequence: no row of the step is another's neighbour
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = first + warp; r < r1; r += 8) {
        float mean, inv;
        warp_row_stats(p.x + (size_t)r * p.width, p.width, p.eps, lane, mean, inv);
        if (lane == 0) {
            stats[r - first][0] = mean;
            stats[r - first][1] = inv;
        }
    }
    __syncthreads();
    const int c0 = blockIdx.y * p.cols, c1 = min(c0 + p.cols, p.width);
    // Columns outermost: a thread keeps, for its column, the taps and the normed values of the last rows in registers (hw[d]: d
    // rows back), so that every row of x is normed once and the weights are read once per tile.  Loops over taps run to the
    // compile-time maximum with the real number as a predicate, which keeps the windows in registers.
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        const float wi = p.w.at(i), bi = p.b.p != nullptr ? p.b.at(i) : 0.f;
        float tw[CONV_MAX_TAPS], hw[CONV_MAX_TAPS];
#pragma unroll
        for (int d = 0; d < CONV_MAX_TAPS; ++d) {
            tw[d] = d < p.n ? p.taps.at(i * p.n + (p.n - 1 - d)) : 0.f;      // the tap that meets the row d back
            hw[d] = 0.f;
        }
        for (int r = first; r < r0; ++r) {                    // the rows before the tile that its taps reach
#pragma unroll
            for (int d = CONV_MAX_TAPS - 1; d > 0; --d) hw[d] = hw[d - 1];
            hw[0] = round_as<TO>((p.x[(size_t)r * p.width + i] - stats[r - first][0]) * stats[r - first][1] * wi + bi);
        }
        for (int row = r0; row < r1; ++row) {
            const int seq = p.row_seq[row];
            TO* yr = (TO*)p.y + (size_t)row * p.width;
#pragma unroll
            for (int d = CONV_MAX_TAPS - 1; d > 0; --d) hw[d] = hw[d - 1];
            hw[0] = round_as<TO>((p.x[(size_t)row * p.width + i] - stats[row - first][0]) * stats[row - first][1] * wi + bi);
            if (seq < 0) {
                fr_store(yr + i, 0.f);
                continue;
            }
            const int t = row - p.seq_start[seq];               // rows of this sequence before this one in the step
            float* hist = p.state + (size_t)p.seq_slots[seq] * p.stride + p.offset;
            float acc = 0.f, seen[CONV_MAX_TAPS];
#pragma unroll
            for (int d = 0; d < CONV_MAX_TAPS; ++d) {
                if (d < p.n) {
                    // d rows back: a row of the step, or, before the step's first row, the history (oldest first)
                    seen[d] = d <= t ? hw[d] : hist[(size_t)(p.n - 1 - (d - t)) * p.width + i];
                    acc = fmaf(tw[d], seen[d], acc);
                } else {
                    seen[d] = 0.f;
                }
            }
            fr_store(yr + i, hw[0] + acc);
            if (p.shift) {                                    // one row per sequence: the history takes it now
#pragma unroll
                for (int d = 0; d < CONV_MAX_TAPS - 1; ++d)
                    if (d < p.n - 1) hist[(size_t)(p.n - 2 - d) * p.width + i] = seen[d];
            }
        }
    }
}

// After norm_conv: the history of every sequence takes the step's last n - 1 rows h (a step of fewer rows keeps the
// youngest of what it had).  A block per sequence and entry where the step brings n - 1 rows or more (every entry is a row of
// the step then); for shorter steps one block per sequence walks the entries in rising order, a thread owning its columns, so
// that nothing is read after it was overwritten.
template <typename TO>
__global__ void __launch_bounds__(256) norm_conv_state_kernel(NormConvArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int seq = blockIdx.x, qlen = p.seq_qlen[seq], first = p.seq_start[seq];
    if (qlen <= 0) return;
    float* hist = p.state + (size_t)p.seq_slots[seq] * p.stride + p.offset;
    const bool alone = qlen < p.n - 1;                        // entries move: this block does them all, in order
    if (alone && blockIdx.y != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float st[2];
    for (int k = alone ? 0 : blockIdx.y; k < (alone ? p.n - 1 : (int)blockIdx.y + 1); ++k) {
        const int s = qlen - (p.n - 1) + k;               // row of the step that becomes entry k; negative: an old entry
        if (s < 0) {
            for (int i = threadIdx.x; i < p.width; i += blockDim.x) hist[(size_t)k * p.width + i] = hist[(size_t)(k + qlen) * p.width + i];
        } else {
            const float* xr = p.x + (size_t)(first + s) * p.width;
            __syncthreads();
            if (warp == 0) {
                float mean, inv;
                warp_row_stats(xr, p.width, p.eps, lane, mean, inv);
                if (lane == 0) {
                    st[0] = mean;
                    st[1] = inv;
                }
            }
            __syncthreads();
            for (int i = threadIdx.x; i < p.width; i += blockDim.x)
                hist[(size_t)k * p.width + i] = round_as<TO>((xr[i] - st[0]) * st[1] * p.w.at(i) + (p.b.p != nullptr ? p.b.at(i) : 0.f));
        }
    }
}

// out = x + half * (a / rms(a) * wa + b / rms(b) * wb): two results side by side, each normed over the width
__global__ void __launch_bounds__(256)
rms_pair_add_kernel(const float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b, FrVec wa, FrVec wb, float eps,
                    float mult, float* __restrict__ out, int width) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t base = (size_t)blockIdx.x * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float u = a[base + i], v = b[base + i];
        sa = fmaf(u, u, sa);
        sb = fmaf(v, v, sb);
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, partial) / (float)width + eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, partial) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[base + i] = x[base + i] + mult * (a[base + i] * ia * wa.at(i) + b[base + i] * ib * wb.at(i));
}

}  // namespace

FR_EXPORT int residual_embed_pair(const int* tokens, const int* row_seq, const int* row_pos, const int* seq_start, const int* seq_qlen,
                                  const int* seq_slots, const void* table, const void* pairs, int table_dtype, int* state, float* out,
                                  int n_rows, int width, int vocab, int buckets, long long mul_prev, long long mul_cur, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (buckets <= 0) FR_REFUSE("embed_pair: %d buckets", buckets);
    if (table_dtype == FR_F32)
        FR_CUDA(fr_launch(embed_pair_kernel<float>, dim3(n_rows), dim3(256), 0, stream, tokens, row_seq, row_pos, seq_start, seq_qlen, seq_slots,
                          (const float*)table, (const float*)pairs, state, out, width, vocab, buckets, mul_prev, mul_cur));
    else if (table_dtype == FR_BF16)
        FR_CUDA(fr_launch(embed_pair_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, tokens, row_seq, row_pos, seq_start, seq_qlen, seq_slots,
                          (const bf16*)table, (const bf16*)pairs, state, out, width, vocab, buckets, mul_prev, mul_cur));
    else FR_REFUSE("embed_pair: unknown dtype %d", table_dtype);
    FR_CHECK_LAUNCH("embed_pair");
    return FR_OK;
}

// x [rows][width] fp32 -> y in out_dtype; w, b (null: none) of w_dtype; taps [width][n] of taps_dtype; the history of a
// sequence is (n - 1) * width floats at state + slot * stride + offset.  shift: every sequence brings exactly one row (the
// history moves on in the kernel; otherwise call residual_norm_conv_state next).
FR_EXPORT int residual_norm_conv(const float* x, const void* w, const void* b, int w_dtype, const void* taps, int taps_dtype, int n, void* y,
                                 int out_dtype, float* state, long long stride, long long offset, const int* row_seq, const int* seq_start,
                                 const int* seq_slots, int n_rows, int width, float eps, int shift, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (n < 1 || n > CONV_MAX_TAPS) FR_REFUSE("norm_conv: %d taps (1 to %d)", n, CONV_MAX_TAPS);
    NormConvArgs p;
    p.x = x; p.w = FrVec{w, w_dtype}; p.b = FrVec{b, w_dtype}; p.taps = FrVec{taps, taps_dtype}; p.y = y; p.state = state; p.stride = stride;
    p.offset = offset; p.row_seq = row_seq; p.seq_start = seq_start; p.seq_qlen = nullptr; p.seq_slots = seq_slots; p.width = width; p.n = n;
    p.shift = shift ? 1 : 0; p.eps = eps; p.rows = n_rows;
    // many rows: tiles of rows with all columns; few rows: a row per block and the columns spread over eight blocks
    p.tile = n_rows >= 512 ? CONV_TILE : 1;
    int splits = n_rows >= 512 ? 1 : (n_rows >= 64 ? 2 : 8);
    if (width < 256 * splits) splits = (width + 255) / 256;
    p.cols = ((width + splits - 1) / splits + 3) / 4 * 4;
    const dim3 grid((n_rows + p.tile - 1) / p.tile, (width + p.cols - 1) / p.cols);
    if (out_dtype == FR_F32) FR_CUDA(fr_launch(norm_conv_kernel<float>, grid, dim3(256), 0, stream, p));
    else if (out_dtype == FR_BF16) FR_CUDA(fr_launch(norm_conv_kernel<bf16>, grid, dim3(256), 0, stream, p));
    else FR_REFUSE("norm_conv: unknown dtype %d", out_dtype);
    FR_CHECK_LAUNCH("norm_conv");
    return FR_OK;
}

FR_EXPORT int residual_norm_conv_state(const float* x, const void* w, const void* b, int w_dtype, int n, int out_dtype, float* state,
                                       long long stride, long long offset, const int* seq_start, const int* seq_qlen, const int* seq_slots,
                                       int n_seqs, int width, float eps, cudaStream_t stream) {
    if (n_seqs <= 0 || n <= 1) return FR_OK;
    if (n > CONV_MAX_TAPS) FR_REFUSE("norm_conv: %d taps (1 to %d)", n, CONV_MAX_TAPS);
    NormConvArgs p;
    p.x = x; p.w = FrVec{w, w_dtype}; p.b = FrVec{b, w_dtype}; p.taps = FrVec{nullptr, 0}; p.y = nullptr; p.state = state; p.stride = stride;
    p.offset = offset; p.row_seq = nullptr; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_slots = seq_slots; p.width = width; p.n = n;
    p.shift = 0; p.eps = eps; p.rows = 0; p.tile = 1; p.cols = width;
    const dim3 grid(n_seqs, n - 1);
    if (out_dtype == FR_F32) FR_CUDA(fr_launch(norm_conv_state_kernel<float>, grid, dim3(256), 0, stream, p));
    else if (out_dtype == FR_BF16) FR_CUDA(fr_launch(norm_conv_state_kernel<bf16>, grid, dim3(256), 0, stream, p));
    else FR_REFUSE("norm_conv: unknown dtype %d", out_dtype);
    FR_CHECK_LAUNCH("norm_conv_state");
    return FR_OK;
}

FR_EXPORT int residual_rms_pair_add(const float* x, const float* a, const float* b, const void* wa, const void* wb, int w_dtype, float eps,
                                    float mult, float* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FR_CUDA(fr_launch(rms_pair_add_kernel, dim3(n_rows), dim3(256), 0, stream, x, a, b, FrVec{wa, w_dtype}, FrVec{wb, w_dtype}, eps, mult, out, width));
    FR_CHECK_LAUNCH("rms_pair_add");
    return FR_OK;
}
