// The delta rule: a mixer whose state per head is a matrix S [dk][dv] that every token first decays, then corrects
// towards its value along its key, then reads with its query:
//
//     S <- diag(g_t) S            g_t one number per head, or one per head and key channel
//     u_t = beta_t (v_t - S^T k_t)
//     S <- S + k_t u_t^T
//     o_t = S^T q_t               (the read sees the present token's write)
//
// and the kernels around it:
//
//   conv_prepare   q, k, v channels of the stacked projection pass a short causal convolution over time (taps per
//                  channel, the last tap is the present token's; the taps-1 inputs before a step's first row come from
//                  the sequence's state, zeros at a sequence's start), then silu; every q and k head is made a unit
//                  vector x / sqrt(sum x^2 + unit_eps), q is multiplied by q_scale.  Results are fp32.
//   conv_state     the last taps-1 inputs of every sequence become its state's history (after conv_prepare has read it)
//   scan           the recurrence, per (sequence, head): up to sixteen threads share one value channel (a column of S, each
//                  with its share of the dk numbers in registers); other warps of the block stage the next eight tokens through shared
//                  memory meanwhile.  beta = sigmoid(raw),
//                  g = exp(-exp(A_log) * softplus(raw + dt_bias)) are formed here in fp32.  Columns of S never mix, so
//                  any split of the value channels over blocks is exact.
//
// State of a sequence: [taps-1][channels] history (channel order of the stacked projection: q, k, v), then the heads'
// matrices [heads][dk][dv], all fp32.  Everything here is fp32 arithmetic; only the projection's rows may be bf16.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* delta_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int MAX_TAPS = 8;

struct ConvArgs {
    const void* x;            // [rows][ld]: q channels at q_off, k at k_off, v at v_off
    const void* taps_w;       // [channels][taps] in channel order q, k, v
    int w_dtype;
    float* out;               // [rows][channels] fp32
    float* state;             // [slots][state_stride], history at offset 0
    long long state_stride;
    const int* row_seq;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_slots;
    int ld, q_off, k_off, v_off, qk_heads, dk, v_channels, taps, rows;
    float q_scale, unit_eps;
    int shift;                // 1: every sequence brings one row, and the thread that convolves a channel moves its history on
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// convolution + silu of channel c (index into q|k|v) at `row`, whose sequence starts at row r0 with history `hist`
template <typename T>
__device__ __forceinline__ float conv_at(const ConvArgs& p, const T* x, int src_col, int c, int row, int r0, const float* hist,
                                         int channels) {
    const FrVec w{p.taps_w, p.w_dtype};
    float acc = 0.f;
    for (int j = 0; j < p.taps; ++j) {
        const int back = p.taps - 1 - j;                 // rows before the present one
        const int r = row - back;
        float in;
        if (r >= r0) in = fr_load(x + (size_t)r * p.ld + src_col);
        else in = hist[(size_t)(p.taps - 1 + (r - r0)) * channels + c];
        acc = fmaf(w.at(c * p.taps + j), in, acc);
    }
    if (p.shift) {
        // one row per sequence: nobody else reads or writes this channel's history, so it moves on here
        float* h = const_cast<float*>(hist);
        const int keep = p.taps - 1;
        float next[MAX_TAPS];
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j)
            if (j < keep) next[j] = j + 1 < keep ? h[(size_t)(j + 1) * channels + c] : fr_load(x + (size_t)row * p.ld + src_col);
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j)
            if (j < keep) h[(size_t)j * channels + c] = next[j];
    }
    return silu_f(acc);
}

// One block per row.  Warps take the q and k heads in turn (a head's channels over the lanes, then the unit norm),
// then all threads take the v channels.
template <typename T>
__global__ void __launch_bounds__(256) conv_prepare_kernel(ConvArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int seq = p.row_seq[row];
    if (seq < 0) return;
    const int r0 = p.seq_start[seq];
    const int qk = p.qk_heads * p.dk, channels = 2 * qk + p.v_channels;
    const float* hist = p.state + (size_t)p.seq_slots[seq] * p.state_stride;
    const T* x = (const T*)p.x;
    float* out = p.out + (size_t)row * channels;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // few rows: the heads and value channels of a row are spread over gridDim.y blocks
    for (int item = blockIdx.y * warps + warp; item < 2 * p.qk_heads; item += gridDim.y * warps) {
        const bool is_q = item < p.qk_heads;
        const int head = is_q ? item : item - p.qk_heads;
        const int c0 = item * p.dk;                                  // channel index in q|k|v order
        const int src0 = (is_q ? p.q_off : p.k_off) + head * p.dk;
        float vals[8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            vals[i] = 0.f;
            if (d < p.dk) {
                vals[i] = conv_at(p, x, src0 + d, c0 + d, row, r0, hist, channels);
                ss = fmaf(vals[i], vals[i], ss);
            }
        }
        ss = fr_warp_sum(ss);
        const float inv = (is_q ? p.q_scale : 1.0f) / sqrtf(ss + p.unit_eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < p.dk) out[c0 + d] = vals[i] * inv;
        }
    }
    for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < p.v_channels; d += gridDim.y * blockDim.x)
        out[2 * qk + d] = conv_at(p, x, p.v_off + d, 2 * qk + d, row, r0, hist, channels);
}

// One block column per sequence: the history becomes the last taps-1 inputs of the sequence, this step's rows included.
template <typename T>
__global__ void __launch_bounds__(256) conv_state_kernel(ConvArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int seq = blockIdx.x;
    const int r0 = p.seq_start[seq], n = p.seq_qlen[seq];
    if (n <= 0 || p.row_seq[r0] < 0) return;
    const int qk = p.qk_heads * p.dk, channels = 2 * qk + p.v_channels;
    float* hist = p.state + (size_t)p.seq_slots[seq] * p.state_stride;
    const T* x = (const T*)p.x;
    const int keep = p.taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        const int src = c < qk ? p.q_off + c : (c < 2 * qk ? p.k_off + (c - qk) : p.v_off + (c - 2 * qk));
        float next[MAX_TAPS];
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j < keep) {
                const int idx = n - keep + j;            // row of the step, counted from the sequence's first row
                next[j] = idx >= 0 ? fr_load(x + (size_t)(r0 + idx) * p.ld + src) : hist[(size_t)(j + n) * channels + c];
            }
        }
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j)
            if (j < keep) hist[(size_t)j * channels + c] = next[j];
    }
}

struct ScanArgs {
    const float* qkv;         // [rows][channels] from conv_prepare: q heads, k heads, v heads
    const void* a_raw;        // [rows][ld_a]: per head, or per head and key channel (per_channel)
    const void* b_raw;        // [rows][ld_b]: per head
    int raw_dtype;
    const void* a_log;        // [heads]
    const void* dt_bias;      // [heads] or [heads * dk]
    int vec_dtype;
    float* out;               // [rows][heads * dv]
    float* state;             // [slots][state_stride]; S of head h at s_off + h * dk * dv, laid out [dk][dv]
    long long state_stride, s_off;
    const int* row_seq;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_slots;
    int ld_a, ld_b, heads, qk_heads, dk, dv, cols, per_channel;
};

constexpr int SCAN_TOKENS = 8;

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <typename TR>
__device__ __forceinline__ float raw_at(const void* p, size_t i) { return fr_load((const TR*)p + i); }

constexpr int STAGE_THREADS = 128;   // warps that only stage tokens, beside the warps that own value channels
// Threads that share a value channel, each with its share of the key channels in registers.  Four: with sixteen (eight
// numbers of 128 per thread, four shuffles per sum) a prompt's scan took as long and a one-token step longer.
constexpr int parts_of(int) { return 4; }

// The first PARTS * p.cols threads walk the tokens: lanes (part, channel) of a warp own 32 / PARTS value channels, PARTS
// lanes each, with the key channels dealt out in groups of four (part p owns groups p, p + PARTS, ...: neighbouring lanes
// read neighbouring 16-byte pieces of shared memory); what the state holds along the key, and the read-out, are summed
// over the PARTS lanes with shuffles.  The other STAGE_THREADS threads stage the next SCAN_TOKENS tokens (q, k, decays, betas, values) into
// the other half of shared memory meanwhile, so that the chain never waits for global memory.  One barrier per SCAN_TOKENS
// tokens.
template <typename TR, int DK, bool PER_CHANNEL>
__global__ void delta_scan_kernel(ScanArgs p) {
    extern __shared__ float sm[];
    constexpr int G_FLOATS = PER_CHANNEL ? SCAN_TOKENS * DK : SCAN_TOKENS;
    constexpr int PARTS = parts_of(DK), CPW = 32 / PARTS;      // lanes per value channel, value channels per warp
    constexpr int PER = DK / PARTS;                   // key channels per thread
    const int buf_floats = 2 * SCAN_TOKENS * DK + G_FLOATS + SCAN_TOKENS + SCAN_TOKENS * p.cols;
    const int seq = blockIdx.x, head = blockIdx.y;
    const int walkers = PARTS * p.cols;
    const bool consumer = (int)threadIdx.x < walkers;
    const int lane = threadIdx.x & 31, part = lane / CPW;
    const int local_col = (threadIdx.x >> 5) * CPW + (lane % CPW);
    const int col = blockIdx.z * p.cols + local_col;
    const bool live_col = consumer && col < p.dv;
    const int r0 = p.seq_start[seq], n = p.seq_qlen[seq];
    fr_pdl_wait();
    fr_pdl_launch();
    if (n <= 0 || p.row_seq[r0] < 0) return;
    const int group = head / (p.heads / p.qk_heads);
    const int qk = p.qk_heads * p.dk, channels = 2 * qk + p.heads * p.dv;
    float* S = p.state + (size_t)p.seq_slots[seq] * p.state_stride + p.s_off + (size_t)head * p.dk * p.dv;
    float s[PER];                                     // s[4 m + e]: key channel 4 (PARTS m + part) + e
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = 4 * (PARTS * (j >> 2) + part) + (j & 3);
        s[j] = (live_col && i < p.dk) ? S[(size_t)i * p.dv + col] : 0.f;
    }
    const FrVec alog{p.a_log, p.vec_dtype}, dtb{p.dt_bias, p.vec_dtype};
    const float rate = expf(alog.at(head));
    const int chunks = (n + SCAN_TOKENS - 1) / SCAN_TOKENS;
    const int n_cols = min(p.cols, p.dv - (int)blockIdx.z * p.cols);

    // stages tokens [t0, t0 + nt) into buffer b: thread `who` of the STAGE_THREADS staging threads.  All of a thread's
    // loads are issued before any of them is used, so that a chunk costs one trip to memory, not one per element.
    auto stage = [&](int t0, int b, int who) {
        float* sq = sm + (size_t)b * buf_floats;
        float* sk = sq + SCAN_TOKENS * DK;
        float* sg = sk + SCAN_TOKENS * DK;
        float* sb = sg + G_FLOATS;
        float* sv = sb + SCAN_TOKENS;
        const int nt = min(SCAN_TOKENS, n - t0);
        constexpr int N_IT = (SCAN_TOKENS * DK + STAGE_THREADS - 1) / STAGE_THREADS;
        float qv[N_IT], kv[N_IT], gz[N_IT];
#pragma unroll
        for (int it = 0; it < N_IT; ++it) {
            const int idx = who + it * STAGE_THREADS;
            const int t = idx / DK, i = idx - t * DK;
            const size_t row = (size_t)(r0 + t0 + t);
            qv[it] = 0.f; kv[it] = 0.f; gz[it] = 0.f;
            if (t < nt && i < p.dk) {
                qv[it] = p.qkv[row * channels + group * p.dk + i];
                kv[it] = p.qkv[row * channels + qk + group * p.dk + i];
                if (PER_CHANNEL) gz[it] = raw_at<TR>(p.a_raw, row * p.ld_a + head * p.dk + i);
            }
        }
        constexpr int N_V = (SCAN_TOKENS * 32 + STAGE_THREADS - 1) / STAGE_THREADS;     // at most 32 value channels per block
        float vv[N_V];
#pragma unroll
        for (int it = 0; it < N_V; ++it) {
            const int idx = who + it * STAGE_THREADS;
            const int t = idx / p.cols, c = idx - t * p.cols;
            vv[it] = (t < nt && c < n_cols) ? p.qkv[(size_t)(r0 + t0 + t) * channels + 2 * qk + head * p.dv + blockIdx.z * p.cols + c] : 0.f;
        }
        float zb = 0.f, za = 0.f;
        if (who < nt) {
            const size_t row = (size_t)(r0 + t0 + who);
            zb = raw_at<TR>(p.b_raw, row * p.ld_b + head);
            if (!PER_CHANNEL) za = raw_at<TR>(p.a_raw, row * p.ld_a + head);
        }
#pragma unroll
        for (int it = 0; it < N_IT; ++it) {
            const int idx = who + it * STAGE_THREADS;
            const int t = idx / DK, i = idx - t * DK;
            if (t < nt) {
                sq[idx] = qv[it];
                sk[idx] = kv[it];
                if (PER_CHANNEL) sg[idx] = i < p.dk ? expf(-rate * softplus_f(gz[it] + dtb.at(head * p.dk + i))) : 1.f;
            }
        }
#pragma unroll
        for (int it = 0; it < N_V; ++it) {
            const int idx = who + it * STAGE_THREADS;
            if (idx < nt * p.cols) sv[idx] = vv[it];
        }
        if (who < nt) {
            sb[who] = 1.0f / (1.0f + expf(-zb));
            if (!PER_CHANNEL) sg[who] = expf(-rate * softplus_f(za + dtb.at(head)));
        }
    };

    if (!consumer) stage(0, 0, threadIdx.x - walkers);
    __syncthreads();
    for (int c = 0; c < chunks; ++c) {
        const int t0 = c * SCAN_TOKENS, nt = min(SCAN_TOKENS, n - t0);
        if (!consumer) {
            if (c + 1 < chunks) stage(t0 + SCAN_TOKENS, (c + 1) & 1, threadIdx.x - walkers);
        } else {
            const float* sq = sm + (size_t)(c & 1) * buf_floats;
            const float* sk = sq + SCAN_TOKENS * DK;
            const float* sg = sk + SCAN_TOKENS * DK;
            const float* sb = sg + G_FLOATS;
            const float* sv = sb + SCAN_TOKENS;
            // one token: the state decays, is corrected along the key, and is read; returns this thread's channel of the result
            auto token = [&](int t) {
                const float4* q4 = (const float4*)(sq + t * DK) + part;
                const float4* k4 = (const float4*)(sk + t * DK) + part;
                const float4* g4 = (const float4*)(sg + t * DK) + part;
                const float gh = PER_CHANNEL ? 1.f : sg[t];
                float4 kk[PER / 4];
                float r = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
                for (int m = 0; m < PER / 4; ++m) {
                    const float4 k = k4[PARTS * m];
                    kk[m] = k;
                    if (PER_CHANNEL) {
                        const float4 g = g4[PARTS * m];
                        s[4 * m] *= g.x; s[4 * m + 1] *= g.y; s[4 * m + 2] *= g.z; s[4 * m + 3] *= g.w;
                    } else {
                        s[4 * m] *= gh; s[4 * m + 1] *= gh; s[4 * m + 2] *= gh; s[4 * m + 3] *= gh;
                    }
                    r = fmaf(k.x, s[4 * m], r);
                    r1 = fmaf(k.y, s[4 * m + 1], r1);
                    r2 = fmaf(k.z, s[4 * m + 2], r2);
                    r3 = fmaf(k.w, s[4 * m + 3], r3);
                }
                r = (r + r1) + (r2 + r3);
#pragma unroll
                for (int w = CPW; w < 32; w <<= 1) r += __shfl_xor_sync(0xffffffffu, r, w);
                const float u = sb[t] * (sv[t * p.cols + local_col] - r);
                float o = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int m = 0; m < PER / 4; ++m) {
                    const float4 k = kk[m], q = q4[PARTS * m];
                    s[4 * m] = fmaf(k.x, u, s[4 * m]);         o = fmaf(q.x, s[4 * m], o);
                    s[4 * m + 1] = fmaf(k.y, u, s[4 * m + 1]); o1 = fmaf(q.y, s[4 * m + 1], o1);
                    s[4 * m + 2] = fmaf(k.z, u, s[4 * m + 2]); o2 = fmaf(q.z, s[4 * m + 2], o2);
                    s[4 * m + 3] = fmaf(k.w, u, s[4 * m + 3]); o3 = fmaf(q.w, s[4 * m + 3], o3);
                }
                o = (o + o1) + (o2 + o3);
#pragma unroll
                for (int w = CPW; w < 32; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
                return o;
            };
            float* out_at = p.out + (size_t)(r0 + t0) * ((size_t)p.heads * p.dv) + head * p.dv + col;
            if (DK <= 128) {
                // the chunk's tokens unrolled, their results kept in registers and stored at the end: a token's read-out
                // (its sums over the lanes, its store) overlaps the next token's chain, and the loads from shared memory
                // run ahead (a store in between would hold them back)
                float res[SCAN_TOKENS];
#pragma unroll
                for (int t = 0; t < SCAN_TOKENS; ++t)
                    if (t < nt) res[t] = token(t);
#pragma unroll
                for (int t = 0; t < SCAN_TOKENS; ++t)
                    if (t < nt && part == 0 && live_col) out_at[(size_t)t * p.heads * p.dv] = res[t];
            } else {
                for (int t = 0; t < nt; ++t) {
                    const float o = token(t);
                    if (part == 0 && live_col) out_at[(size_t)t * p.heads * p.dv] = o;
                }
            }
        }
        __syncthreads();
    }
    if (live_col) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = 4 * (PARTS * (j >> 2) + part) + (j & 3);
            if (i < p.dk) S[(size_t)i * p.dv + col] = s[j];
        }
    }
}

template <typename TR, int DK>
int launch_scan(const ScanArgs& p, int n_seqs, int splits, cudaStream_t stream) {
    const size_t floats = (size_t)2 * SCAN_TOKENS * DK + (p.per_channel ? (size_t)SCAN_TOKENS * DK : SCAN_TOKENS) + SCAN_TOKENS +
                          (size_t)SCAN_TOKENS * p.cols;
    const size_t smem = 2 * floats * sizeof(float);
    const dim3 grid(n_seqs, p.heads, splits);
    const dim3 block(parts_of(DK) * p.cols + STAGE_THREADS);
    if (p.per_channel) {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(delta_scan_kernel<TR, DK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(delta_scan_kernel<TR, DK, true>, grid, block, smem, stream, p));
    } else {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(delta_scan_kernel<TR, DK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(delta_scan_kernel<TR, DK, false>, grid, block, smem, stream, p));
    }
    FR_CHECK_LAUNCH("delta scan");
    return FR_OK;
}

template <typename TR>
int scan_by_size(const ScanArgs& p, int n_seqs, int splits, cudaStream_t stream) {
    if (p.dk <= 16) return launch_scan<TR, 16>(p, n_seqs, splits, stream);
    if (p.dk <= 32) return launch_scan<TR, 32>(p, n_seqs, splits, stream);
    if (p.dk <= 64) return launch_scan<TR, 64>(p, n_seqs, splits, stream);
    if (p.dk <= 128) return launch_scan<TR, 128>(p, n_seqs, splits, stream);
    if (p.dk <= 256) return launch_scan<TR, 256>(p, n_seqs, splits, stream);
    FR_REFUSE("delta scan: %d key channels per head (at most 256)", p.dk);
}

int fill_conv(ConvArgs& p, const void* x, int ld, int q_off, int k_off, int v_off, const void* taps_w, int w_dtype, float* out,
              float* state, long long state_stride, const int* row_seq, const int* seq_start, const int* seq_qlen,
              const int* seq_slots, int rows, int qk_heads, int dk, int v_channels, int taps, float q_scale, float unit_eps) {
    if (taps < 1 || taps > MAX_TAPS) FR_REFUSE("short convolution: %d taps (1 to %d)", taps, MAX_TAPS);
    if (dk <= 0 || dk > 256 || qk_heads <= 0 || v_channels <= 0) FR_REFUSE("short convolution: %d heads of %d, %d value channels", qk_heads, dk, v_channels);
    p.x = x; p.taps_w = taps_w; p.w_dtype = w_dtype; p.out = out; p.state = state; p.state_stride = state_stride;
    p.row_seq = row_seq; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_slots = seq_slots;
    p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.qk_heads = qk_heads; p.dk = dk; p.v_channels = v_channels;
    p.taps = taps; p.rows = rows; p.q_scale = q_scale; p.unit_eps = unit_eps; p.shift = 0;
    return FR_OK;
}

}  // namespace

// q, k (qk_heads x dk each) and v (v_channels) of x [rows][ld] -> out [rows][2 qk_heads dk + v_channels] fp32.
// shift_history: only where every sequence of the step brings exactly one row; the state's history then moves on in this
// kernel and delta_conv_state is not needed.
FR_EXPORT int delta_conv_prepare(const void* x, int ld, int q_off, int k_off, int v_off, const void* taps_w, int w_dtype, float* out,
                                 const float* state, long long state_stride, const int* row_seq, const int* seq_start,
                                 const int* seq_slots, int rows, int qk_heads, int dk, int v_channels, int taps, float q_scale,
                                 float unit_eps, int shift_history, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    ConvArgs p;
    const int rc = fill_conv(p, x, ld, q_off, k_off, v_off, taps_w, w_dtype, out, (float*)state, state_stride, row_seq, seq_start,
                             nullptr, seq_slots, rows, qk_heads, dk, v_channels, taps, q_scale, unit_eps);
    if (rc != FR_OK) return rc;
    p.shift = shift_history && taps > 1 ? 1 : 0;
    int tiles = 1;
    if (rows < 128) {
        const int work = (2 * qk_heads + 7) / 8 + (v_channels + 255) / 256;      // rounds of a block's warps and threads
        tiles = work < 8 ? work : 8;
        if (tiles < 1) tiles = 1;
    }
    if (dtype == FR_F32) FR_CUDA(fr_launch(conv_prepare_kernel<float>, dim3(rows, tiles), dim3(256), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(conv_prepare_kernel<bf16>, dim3(rows, tiles), dim3(256), 0, stream, p));
    else FR_REFUSE("short convolution: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("conv_prepare");
    return FR_OK;
}

FR_EXPORT int delta_conv_state(const void* x, int ld, int q_off, int k_off, int v_off, float* state, long long state_stride,
                               const int* row_seq, const int* seq_start, const int* seq_qlen, const int* seq_slots, int n_seqs,
                               int qk_heads, int dk, int v_channels, int taps, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0 || taps <= 1) return FR_OK;
    ConvArgs p;
    const int rc = fill_conv(p, x, ld, q_off, k_off, v_off, nullptr, 0, nullptr, state, state_stride, row_seq, seq_start, seq_qlen,
                             seq_slots, 0, qk_heads, dk, v_channels, taps, 1.f, 0.f);
    if (rc != FR_OK) return rc;
    const int channels = 2 * qk_heads * dk + v_channels;
    const dim3 grid(n_seqs, (channels + 255) / 256);
    if (dtype == FR_F32) FR_CUDA(fr_launch(conv_state_kernel<float>, grid, dim3(256), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(conv_state_kernel<bf16>, grid, dim3(256), 0, stream, p));
    else FR_REFUSE("short convolution: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("conv_state");
    return FR_OK;
}

// per_channel 0: a_raw [rows][>= heads], dt_bias [heads]; 1: a_raw [rows][>= heads * dk], dt_bias [heads * dk].
// raw_dtype: dtype of a_raw and b_raw; vec_dtype: dtype of a_log and dt_bias.
FR_EXPORT int delta_scan(const float* qkv, const void* a_raw, int ld_a, const void* b_raw, int ld_b, int raw_dtype, const void* a_log,
                         const void* dt_bias, int vec_dtype, float* out, float* state, long long state_stride, long long s_off,
                         const int* row_seq, const int* seq_start, const int* seq_qlen, const int* seq_slots, int n_seqs, int heads,
                         int qk_heads, int dk, int dv, int per_channel, cudaStream_t stream) {
    if (n_seqs <= 0) return FR_OK;
    if (heads <= 0 || qk_heads <= 0 || heads % qk_heads || dk <= 0 || dv <= 0)
        FR_REFUSE("delta scan: %d heads on %d query/key heads, dk %d, dv %d", heads, qk_heads, dk, dv);
    ScanArgs p;
    p.qkv = qkv; p.a_raw = a_raw; p.b_raw = b_raw; p.raw_dtype = raw_dtype; p.a_log = a_log; p.dt_bias = dt_bias; p.vec_dtype = vec_dtype;
    p.out = out; p.state = state; p.state_stride = state_stride; p.s_off = s_off; p.row_seq = row_seq; p.seq_start = seq_start;
    p.seq_qlen = seq_qlen; p.seq_slots = seq_slots; p.ld_a = ld_a; p.ld_b = ld_b; p.heads = heads; p.qk_heads = qk_heads; p.dk = dk;
    p.dv = dv; p.per_channel = per_channel ? 1 : 0;
    // value channels per block (four threads each): 32, or 16 where the device would otherwise stay empty
    const int sms = fr_sm_count() > 0 ? fr_sm_count() : 128;
    int cols = 32;
    if ((long long)n_seqs * heads * ((dv + cols - 1) / cols) < 2LL * sms) cols = 16;
    if (cols > ((dv + 7) / 8) * 8) cols = ((dv + 7) / 8) * 8;
    p.cols = cols;
    const int splits = (dv + cols - 1) / cols;
    if (raw_dtype == FR_F32) return scan_by_size<float>(p, n_seqs, splits, stream);
    if (raw_dtype == FR_BF16) return scan_by_size<bf16>(p, n_seqs, splits, stream);
    FR_REFUSE("delta scan: unknown dtype %d", raw_dtype);
}

// ------------------------------------------------------------------ the generalized delta rule
// A decay per head and key channel and a removal along the unit key, both reading the old state:
//
//     S <- diag(w_t) S - (a_t * u_t) (u_t^T S) + k_t v_t^T,   o_t = S^T r_t
//
// with u = k / sqrt(sum k^2 + unit_eps) per head, w = exp(-decay_rate * sigmoid(z + z_bias)) and a = sigmoid(a_raw + a_bias),
// all formed in fp32 by `general_prepare` (one warp per row and head), which leaves per row and head five vectors of dk
// floats: w, a * u, u, k, r.  `general_scan` walks the tokens of a sequence: four lanes share a value channel (a column of
// S), each with a quarter of the key channels in registers; the block stages eight tokens at a time through shared memory,
// the next eight loaded into registers before the present ones are walked.  Columns of S never mix, so any split of the value
// channels over blocks is exact.  State of a sequence: [heads][dk][dv] fp32 at `s_off`.
namespace {

struct GeneralPrepArgs {
    const void* proj;        // [rows][ld]: r at r_off, k at k_off (heads * dk each), in the activation dtype
    const float* z;          // [rows][ld_z] fp32: the decay's raw projection
    const float* a_raw;      // [rows][ld_a] fp32: the removal's raw projection
    FrVec z_bias, a_bias;    // [heads * dk]
    float* out;              // [rows][heads][5][dk]
    int ld, r_off, k_off, ld_z, ld_a, heads, dk, rows;
    float rate, unit_eps;
};

template <typename T>
__global__ void __launch_bounds__(128) general_prepare_kernel(GeneralPrepArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= p.rows * p.heads) return;
    const int row = item / p.heads, h = item - row * p.heads;
    const T* x = (const T*)p.proj + (size_t)row * p.ld;
    float ss = 0.f;
    for (int i = lane; i < p.dk; i += 32) {
        const float k = fr_load(x + p.k_off + h * p.dk + i);
        ss = fmaf(k, k, ss);
    }
    const float inv = 1.0f / sqrtf(fr_warp_sum(ss) + p.unit_eps);
    float* o = p.out + (size_t)item * 5 * p.dk;
    for (int i = lane; i < p.dk; i += 32) {
        const int c = h * p.dk + i;
        const float k = fr_load(x + p.k_off + c), r = fr_load(x + p.r_off + c);
        const float zz = p.z[(size_t)row * p.ld_z + c] + p.z_bias.at(c);
        const float aa = p.a_raw[(size_t)row * p.ld_a + c] + p.a_bias.at(c);
        const float u = k * inv;
        o[i] = expf(-p.rate / (1.0f + expf(-zz)));
        o[p.dk + i] = u / (1.0f + expf(-aa));
        o[2 * p.dk + i] = u;
        o[3 * p.dk + i] = k;
        o[4 * p.dk + i] = r;
    }
}

struct GeneralScanArgs {
    const float* prep;       // [rows][heads][5][dk]
    const void* v;           // [rows][ld_v], head h at v_off + h * dv
    float* out;              // [rows][heads * dv]
    float* state;
    long long state_stride, s_off;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_slots;
    int ld_v, v_off, heads, dk, dv, cols;
};

// tokens staged at a time: fewer where a token is wide, so that what a thread holds of the next chunk stays in registers
constexpr int gen_tokens(int dkp, int lpc) { return lpc >= 16 ? (dkp <= 128 ? 8 : 4) : (dkp <= 64 ? 8 : (dkp <= 128 ? 4 : 2)); }

// threads of a block.  (Blocks of 512 threads for the sixteen-lane form, which would share a token's staged vectors among
// 32 columns instead of 8, ran 1.5 times slower: sixteen warps then queue at one SM's shared memory while other SMs idle.)
constexpr int scan_threads(int) { return 128; }

// DKP: key channels rounded up to 16, 32, 64, 128 or 256.  LPC lanes share a value channel (a column of S): 4, or 16 where
// the step has few sequences (a lane's share of a token is then a quarter as long, and four times as many warps fill the
// device); a lane holds DKP / LPC key channels, dealt out in groups of four so that the lanes of a column read neighbouring
// 16-byte pieces of shared memory.
template <typename T, int DKP, int LPC>
__global__ void __launch_bounds__(scan_threads(LPC)) general_scan_kernel(GeneralScanArgs p) {
    extern __shared__ __align__(16) float gsm[];
    constexpr int PER = DKP / LPC, VEC = 5 * DKP, GEN_TOKENS = gen_tokens(DKP, LPC), THREADS = scan_threads(LPC), COLS = THREADS / LPC;
    static_assert(PER >= 4 && PER % 4 == 0, "a lane holds whole groups of four key channels");
    const int seq = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int part = tid % LPC, local_col = tid / LPC, col = blockIdx.z * p.cols + local_col;
    const bool live_col = local_col < p.cols && col < p.dv;
    fr_pdl_wait();
    fr_pdl_launch();
    const int n = p.seq_qlen[seq], r0 = p.seq_start[seq];
    if (n <= 0) return;
    float* S = p.state + (size_t)p.seq_slots[seq] * p.state_stride + p.s_off + (size_t)head * p.dk * p.dv;
    float s[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = 4 * (LPC * (j >> 2) + part) + (j & 3);
        s[j] = (live_col && i < p.dk) ? S[(size_t)i * p.dv + col] : 0.f;
    }
    constexpr int BUF = GEN_TOKENS * (VEC + COLS);
    // what one thread loads of a chunk: vectors (w, a u, u, k, r padded to DKP with zeros) and the block's value channels
    constexpr int N_IT = (GEN_TOKENS * VEC + THREADS - 1) / THREADS, N_V = (GEN_TOKENS * COLS + THREADS - 1) / THREADS;
    float held[N_IT], held_v[N_V];
    const float* prep = p.prep + ((size_t)r0 * p.heads + head) * 5 * p.dk;
    const T* vals = (const T*)p.v + (size_t)r0 * p.ld_v + p.v_off + head * p.dv + blockIdx.z * p.cols;
    auto fetch = [&](int t0) {
        const int nt = min(GEN_TOKENS, n - t0);
#pragma unroll
        for (int it = 0; it < N_IT; ++it) {
            const int idx = tid + it * THREADS;
            const int t = idx / VEC, rest = idx - t * VEC, which = rest / DKP, i = rest - which * DKP;
            held[it] = (idx < GEN_TOKENS * VEC && t < nt && i < p.dk) ? prep[(size_t)(t0 + t) * p.heads * 5 * p.dk + which * p.dk + i] : 0.f;
        }
#pragma unroll
        for (int it = 0; it < N_V; ++it) {
            const int idx = tid + it * THREADS;
            const int t = idx / COLS, c = idx - t * COLS;
            held_v[it] = (idx < GEN_TOKENS * COLS && t < nt && c < p.cols && blockIdx.z * p.cols + c < p.dv)
                             ? fr_load(vals + (size_t)(t0 + t) * p.ld_v + c) : 0.f;
        }
    };
    auto put = [&](int b) {
        float* dst = gsm + (size_t)b * BUF;
#pragma unroll
        for (int it = 0; it < N_IT; ++it) {
            const int idx = tid + it * THREADS;
            if (idx < GEN_TOKENS * VEC) dst[idx] = held[it];
        }
#pragma unroll
        for (int it = 0; it < N_V; ++it) {
            const int idx = tid + it * THREADS;
            if (idx < GEN_TOKENS * COLS) dst[GEN_TOKENS * VEC + idx] = held_v[it];
        }
    };
    const int chunks = (n + GEN_TOKENS - 1) / GEN_TOKENS;
    float* out_at = p.out + (size_t)r0 * ((size_t)p.heads * p.dv) + head * p.dv + col;
    fetch(0);
    put(0);
    __syncthreads();
    for (int c = 0; c < chunks; ++c) {
        const int t0 = c * GEN_TOKENS, nt = min(GEN_TOKENS, n - t0);
        if (c + 1 < chunks) fetch(t0 + GEN_TOKENS);
        const float* buf = gsm + (size_t)(c & 1) * BUF;
        // one token: the state decays, loses its part along the unit key, takes the new pair; returns this lane's share of the read-out
        auto token = [&](int t) {
            const float4* w4 = (const float4*)(buf + t * VEC) + part;
            const float4* b4 = w4 + DKP / 4;
            const float4* u4 = b4 + DKP / 4;
            const float4* k4 = u4 + DKP / 4;
            const float4* r4 = k4 + DKP / 4;
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int m = 0; m < PER / 4; ++m) {
                const float4 u = u4[LPC * m];
                d0 = fmaf(u.x, s[4 * m], d0);
                d1 = fmaf(u.y, s[4 * m + 1], d1);
                d2 = fmaf(u.z, s[4 * m + 2], d2);
                d3 = fmaf(u.w, s[4 * m + 3], d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
#pragma unroll
            for (int o = 1; o < LPC; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float val = buf[GEN_TOKENS * VEC + t * COLS + local_col];
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int m = 0; m < PER / 4; ++m) {
                const float4 w = w4[LPC * m], b = b4[LPC * m], k = k4[LPC * m], r = r4[LPC * m];
                s[4 * m] = fmaf(k.x, val, fmaf(-b.x, dot, w.x * s[4 * m]));
                s[4 * m + 1] = fmaf(k.y, val, fmaf(-b.y, dot, w.y * s[4 * m + 1]));
                s[4 * m + 2] = fmaf(k.z, val, fmaf(-b.z, dot, w.z * s[4 * m + 2]));
                s[4 * m + 3] = fmaf(k.w, val, fmaf(-b.w, dot, w.w * s[4 * m + 3]));
                o0 = fmaf(r.x, s[4 * m], o0);
                o1 = fmaf(r.y, s[4 * m + 1], o1);
                o2 = fmaf(r.z, s[4 * m + 2], o2);
                o3 = fmaf(r.w, s[4 * m + 3], o3);
            }
            return (o0 + o1) + (o2 + o3);
        };
        auto finish = [&](int t, float o) {
#pragma unroll
            for (int x = 1; x < LPC; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (part == 0 && live_col) out_at[(size_t)(t0 + t) * p.heads * p.dv] = o;
        };
        if constexpr (LPC < 16) {
            // the chunk's tokens unrolled, their read-outs summed over the lanes at the end of the chunk, so that a read-out
            // overlaps the next token's chain (measured: 2.34 -> 1.99 ms for 8 x 1,024 tokens; with sixteen lanes it lost)
            float res[GEN_TOKENS];
#pragma unroll
            for (int t = 0; t < GEN_TOKENS; ++t) {
                if (t >= nt) break;
                res[t] = token(t);
            }
#pragma unroll
            for (int t = 0; t < GEN_TOKENS; ++t) {
                if (t >= nt) break;
                finish(t, res[t]);
            }
        } else {
            for (int t = 0; t < nt; ++t) finish(t, token(t));
        }
        if (c + 1 < chunks) put((c + 1) & 1);
        __syncthreads();
    }
    if (live_col) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = 4 * (LPC * (j >> 2) + part) + (j & 3);
            if (i < p.dk) S[(size_t)i * p.dv + col] = s[j];
        }
    }
}

template <typename T, int DKP, int LPC>
int launch_general(GeneralScanArgs p, int n_seqs, cudaStream_t stream) {
    constexpr int COLS = scan_threads(LPC) / LPC;
    p.cols = COLS;
    if (p.cols > ((p.dv + 7) / 8) * 8) p.cols = ((p.dv + 7) / 8) * 8;      // few value channels: the rest of the block only helps to stage
    const size_t smem = (size_t)2 * gen_tokens(DKP, LPC) * (5 * DKP + COLS) * sizeof(float);
    if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(general_scan_kernel<T, DKP, LPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid(n_seqs, p.heads, (p.dv + p.cols - 1) / p.cols);
    FR_CUDA(fr_launch(general_scan_kernel<T, DKP, LPC>, grid, dim3(scan_threads(LPC)), smem, stream, p));
    FR_CHECK_LAUNCH("general delta scan");
    return FR_OK;
}

template <typename T, int DKP>
int general_by_lanes(const GeneralScanArgs& p, int n_seqs, cudaStream_t stream) {
    if constexpr (DKP >= 64) {
        // sixteen lanes per column while four would leave schedulers without a warp (four per SM)
        const int sms = fr_sm_count() > 0 ? fr_sm_count() : 128;
        if ((long long)n_seqs * p.heads * p.dv * 4 / 32 < 8LL * sms) return launch_general<T, DKP, 16>(p, n_seqs, stream);
    }
    return launch_general<T, DKP, 4>(p, n_seqs, stream);
}

template <typename T>
int general_by_size(const GeneralScanArgs& p, int n_seqs, cudaStream_t stream) {
    if (p.dk <= 16) return general_by_lanes<T, 16>(p, n_seqs, stream);
    if (p.dk <= 32) return general_by_lanes<T, 32>(p, n_seqs, stream);
    if (p.dk <= 64) return general_by_lanes<T, 64>(p, n_seqs, stream);
    if (p.dk <= 128) return general_by_lanes<T, 128>(p, n_seqs, stream);
    if (p.dk <= 256) return general_by_lanes<T, 256>(p, n_seqs, stream);
    FR_REFUSE("general delta scan: %d key channels per head (at most 256)", p.dk);
}

}  // namespace

// proj [rows][ld] of `dtype` (r at r_off, k at k_off); z [rows][ld_z] and a_raw [rows][ld_a] fp32; biases [heads * dk] of
// vec_dtype; out [rows][heads][5][dk] fp32 (w, a u, u, k, r)
FR_EXPORT int delta_general_prepare(const void* proj, int ld, int r_off, int k_off, const float* z, int ld_z, const float* a_raw, int ld_a,
                                    const void* z_bias, const void* a_bias, int vec_dtype, float* out, int rows, int heads, int dk, float rate,
                                    float unit_eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (heads <= 0 || dk <= 0) FR_REFUSE("general delta rule: %d heads of %d", heads, dk);
    GeneralPrepArgs p;
    p.proj = proj; p.z = z; p.a_raw = a_raw; p.z_bias = FrVec{z_bias, vec_dtype}; p.a_bias = FrVec{a_bias, vec_dtype}; p.out = out; p.ld = ld;
    p.r_off = r_off; p.k_off = k_off; p.ld_z = ld_z; p.ld_a = ld_a; p.heads = heads; p.dk = dk; p.rows = rows; p.rate = rate; p.unit_eps = unit_eps;
    const dim3 grid((unsigned)(((long long)rows * heads + 3) / 4));
    if (dtype == FR_F32) FR_CUDA(fr_launch(general_prepare_kernel<float>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(general_prepare_kernel<bf16>, grid, dim3(128), 0, stream, p));
    else FR_REFUSE("general delta rule: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("general_prepare");
    return FR_OK;
}

// prep as general_prepare leaves it; v [rows][ld_v] of `dtype`, head h at v_off + h * dv; out [rows][heads * dv] fp32
FR_EXPORT int delta_general_scan(const float* prep, const void* v, int ld_v, int v_off, float* out, float* state, long long state_stride,
                                 long long s_off, const int* seq_start, const int* seq_qlen, const int* seq_slots, int n_seqs, int heads,
                                 int dk, int dv, int dtype, cudaStream_t stream) {
    if (n_seqs <= 0) return FR_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0) FR_REFUSE("general delta scan: %d heads, dk %d, dv %d", heads, dk, dv);
    GeneralScanArgs p;
    p.prep = prep; p.v = v; p.out = out; p.state = state; p.state_stride = state_stride; p.s_off = s_off; p.seq_start = seq_start;
    p.seq_qlen = seq_qlen; p.seq_slots = seq_slots; p.ld_v = ld_v; p.v_off = v_off; p.heads = heads; p.dk = dk; p.dv = dv;
    p.cols = 0;                                      // chosen with the lanes per column
    if (dtype == FR_F32) return general_by_size<float>(p, n_seqs, stream);
    if (dtype == FR_BF16) return general_by_size<bf16>(p, n_seqs, stream);
    FR_REFUSE("general delta scan: unknown dtype %d", dtype);
}
