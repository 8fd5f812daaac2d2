// The operations that parts are made of.  Every one launches this library's own CUDA
// kernels (csrc/) on the Ops object's stream; there is no CPU path, and a kernel library
// that cannot be loaded is an error of the call that needed it.
//
// Memory: results are taken from the Ops object's current Arena, which the caller of a
// pass (the model's run loop) sets and resets; a result lives until the arena that it
// came from is reset.  Weights, cache pools and anything that must outlive a pass are
// allocated by their owners with DeviceBuffer.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "friday/base.h"
#include "friday/parts.h"

struct GemmFusion;          // csrc/gemm_tc_fusion.h: optional work at the two ends of the tensor-core product

namespace friday {

void cuda_check(cudaError_t e, const char* what);

class DeviceBuffer {
public:
    DeviceBuffer() {}
    explicit DeviceBuffer(size_t bytes, bool zero = false);
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void* get() const { return p_; }
    size_t bytes() const { return n_; }
    template <class T> T* as() const { return (T*)p_; }

private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// Hands out device memory by bumping an offset; reset() takes everything back.  When a block runs out,
// another is added (earlier results stay where they are); the next reset() joins the blocks into one, after
// which addresses differ from before: generation() counts those events, so that whoever keeps addresses (a
// captured graph) knows when they are stale.
class Arena {
public:
    explicit Arena(cudaStream_t stream, size_t first_block = (size_t)1 << 20) : stream_(stream), first_(first_block) {}
    ~Arena();
    void* alloc(size_t bytes);
    void reset();
    uint64_t generation() const { return generation_; }
    size_t capacity() const;
    bool frozen = false;            // true while a graph is being captured: growing is an error then

private:
    struct BlockMem { void* p; size_t size; };
    std::vector<BlockMem> blocks_;
    size_t offset_ = 0;             // in the last block
    cudaStream_t stream_;
    size_t first_;
    uint64_t generation_ = 0;
};

// Rows on their way from one product to the next.  Plain rows are a tensor.  Deferred rows are rows whose
// RMSNorm the product that made them has begun: `t` holds weight (*) x rounded to bf16, `ssq` [parts, rows]
// each part's share of the rows' sums of squares; the product that takes them finishes the norm by scaling
// its own rows with 1 / sqrt(sum / width + eps).  Anything else asks Ops::materialize, which runs the norm's
// kernel on `source`.
struct Rows {
    Tensor t;
    bool deferred = false;
    Tensor ssq, source, weight;
    float eps = 0;
    Rows() {}
    Rows(const Tensor& x) : t(x) {}
};

struct PartOut {
    Tensor x;                // residual + part(h)
    bool has_normed = false;
    Rows normed;             // `then` of x, if the part produced it
    PartOut() {}
    PartOut(const Tensor& t) : x(t) {}
    PartOut(const Tensor& t, const Rows& n) : x(t), has_normed(true), normed(n) {}
};


class Ops {
public:
    Ops(int device, cudaStream_t stream);
    ~Ops();
    Ops(const Ops&) = delete;

    int device() const { return device_; }
    cudaStream_t stream() const { return stream_; }
    int sm_count() const { return sms_; }
    Arena* arena = nullptr;                                   // where results come from
    Tensor alloc(DType dtype, int64_t rows, int64_t cols);
    float* scratch_floats(int64_t n);                         // from the arena

    // ---- row-wise
    Tensor embedding(const int* tokens, int64_t n, const Tensor& table, Tensor* out = nullptr);
    Tensor gather_rows(const int* rows, int64_t n, const Tensor& src);
    Tensor rmsnorm(const Tensor& x, const Tensor& weight, float eps, Tensor* out = nullptr);
    // columns alternate gate, up; act 1: silu(gate) * up, act 2: gelu_tanh(gate) * up
    Tensor swiglu(const Tensor& gate_up, int act = 1);
    // Rotates q and k inside qkv [rows, (nq + 2 nkv) * hd] (denominators null: no rotation) and, if the view
    // may be written, stores k and v in the cache rows of (row_seq, row_pos).
    void rope_kv_write(Tensor& qkv, const int* row_seq, const int* row_pos, const float* denominators, int rotary_dim,
                       int n_heads, int n_kv_heads, int head_dim, const CacheView* view);
    void advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws, int n);
    void scale_rows(Tensor& x, float scale);                  // x *= scale (embedding multipliers)
    void finish_logits(Tensor& logits, const Tensor* bias, float scale, float softcap);

    // ---- a residual stream in 32-bit floats beside activations in another dtype
    // y = x / sqrt(mean(x^2) + eps) * (offset + weight), x and y in dtypes of their own
    Tensor rmsnorm_to(const Tensor& x, const Tensor& weight, float offset, float eps, DType out_dtype);
    Tensor concat_cast(const Tensor& a, const Tensor& b, DType out_dtype);            // [a, b] side by side
    // residual (fp32) + alpha * y (+ beta * z): a new fp32 tensor, or `residual` itself with in_place
    Tensor add_scaled(const Tensor& residual, const Tensor& y, float alpha, const Tensor* z = nullptr, float beta = 0.f,
                      bool in_place = false);
    // residual + alpha * (x weight^T + bias): in the product's epilogue where residual and result share a dtype and
    // alpha is 1; otherwise the product in 32-bit and add_scaled
    Tensor linear_residual(const Rows& x, const Tensor& weight, const Tensor* bias, const Tensor& residual, float alpha = 1.0f);
    // y = (x - mean) / sqrt(variance + eps) * weight + bias (bias null: none), x and y in dtypes of their own
    Tensor layernorm_to(const Tensor& x, const Tensor& weight, const Tensor* bias, float eps, DType out_dtype);
    // table[token] * scale as 32-bit rows: the start of a 32-bit residual stream, without a rounding in between
    Tensor embed_rows(const int* tokens, int64_t n, const Tensor& table, float scale);
    // table[token] + positions[row_pos] as 32-bit rows: a learned position table beside the token table
    Tensor embed_pos_rows(const StepContext& ctx, const Tensor& table, const Tensor& positions);
    // y = h + (h_before - h) * shift with h = x / sqrt(mean(x^2) + eps) * weight (x: the 32-bit stream) and h_before the h of
    // the row before in the sequence; the h before a step's first row comes from the state (`view`: a state of at least
    // the width per sequence), which then keeps the h of the step's last row
    Tensor norm_shift(const Tensor& x, const Tensor& weight, float eps, const Tensor& shift, const CacheView& view, const StepContext& ctx,
                      DType out_dtype);
    // x + mult * y / sqrt(mean(y^2) + eps) * weight (x, y 32-bit); with next_weight also the norm of that sum in `next_dtype`
    // (what the sublayer after it reads), returned through `next`
    Tensor post_norm_add(const Tensor& x, const Tensor& y, const Tensor& weight, float eps, float mult, const Tensor* next_weight = nullptr,
                         float next_eps = 0.f, DType next_dtype = DType::F32, Tensor* next = nullptr);
    // in place: z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2; pq = (p, q)
    void two_sided_act(Tensor& z, const Tensor& pq);
    // keys [n_kv_heads][head_dim] at column k_off and values [n_kv_heads][v_head_dim] at column v_off of every row of
    // `src` go to the cache rows of (row_seq, row_pos)
    void kv_store(const Tensor& src, int64_t k_off, int64_t v_off, const CacheView& view, const StepContext& ctx);
    // the per-layer token input, in place on the 32-bit stream x: e = table[token][col0 .. col0 + dim);
    // y = proj (gelu_tanh(gate x) * e); x += y / sqrt(mean(y^2) + eps) * norm
    void token_input(Tensor& x, const StepContext& ctx, const Tensor& table, int64_t col0, const Tensor& gate, const Tensor& proj,
                     const Tensor& norm, float eps);

    // table[token] + pairs[(previous token * mul_prev + token * mul_cur) mod buckets] as 32-bit rows, the table's last row
    // (number `buckets`) for a sequence's first token; the token before a step's first row comes from `view` (a state of one
    // int32 per sequence), which then keeps the step's last token
    Tensor embed_pair_rows(const StepContext& ctx, const Tensor& table, const Tensor& pairs, int64_t buckets, int64_t mul_prev,
                           int64_t mul_cur, const CacheView& view);
    // h + conv(h) with h = layer_norm(x) (bias null: none) in `out_dtype` and conv(h)_t = sum_j taps[:, j] h_(t - n + 1 + j) for
    // taps [width, n], zeros before a sequence's start; `view` is a state of (n - 1) * width floats per sequence: its last
    // n - 1 rows h, which the step's last rows replace
    Tensor norm_conv(const Tensor& x, const Tensor& weight, const Tensor* bias, float eps, const Tensor& taps, const CacheView& view,
                     const StepContext& ctx, DType out_dtype);
    // x + mult * (a / rms(a) * wa + b / rms(b) * wb), all rows 32-bit: two results side by side, each normed over the width
    Tensor rms_pair_add(const Tensor& x, const Tensor& a, const Tensor& b, const Tensor& wa, const Tensor& wb, float eps, float mult);

    // ---- mixers with a matrix state per head (csrc/recurrence.cu)
    // out [n][rows, width]: row + (row before - row) * mu[s]; the row before a step's first comes from the state
    Tensor shift_mix(const Tensor& h, const std::vector<Tensor>& mu, const CacheView& view, const StepContext& ctx);
    void tanh_rows(Tensor& x);
    struct ScanSpec {
        int heads = 0, dk = 0, dv = 0;
        int mode = 0;                   // 0: a = sigmoid(z)^(1/tau); 1: a = exp(-exp(z))
        float q_scale = 1.f, tau = 1.f;
        int64_t state_offset = 0;       // floats before the heads' matrices in a sequence's state
        const Tensor* z_bias = nullptr; // [heads * dk]
        const Tensor* bonus = nullptr;  // [heads * dk]: read the state before the update, with bonus * k v^T for the present token
        const Tensor* carry = nullptr;  // rows whose last one per sequence is kept at the start of the state
    };
    // q, k [rows, >= heads * dk], v [rows, >= heads * dv] (the tensors' row strides are used), z [rows, heads * dk] fp32
    Tensor state_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& z, const ScanSpec& spec, const CacheView& view,
                      const StepContext& ctx);
    // o [rows, heads * dv] fp32 -> o / rms_head(o) * weight * silu(gate) * out_scale in `dtype`
    // gate_sigmoid: the gate passes a sigmoid instead of silu
    Tensor head_norm_gate(const Tensor& o, const Tensor& gate, const Tensor& weight, bool weight_per_head, int heads, int dv,
                          float eps, float out_scale, DType dtype, const StepContext& ctx, bool gate_sigmoid = false);

    // ---- the delta rule (csrc/delta.cu): a state per head that every token decays, corrects along its key and reads
    struct DeltaSpec {
        int heads = 0, qk_heads = 0, dk = 0, dv = 0, taps = 1;
        bool per_channel = false;       // a decay per head and key channel instead of one per head
        float q_scale = 1.f, unit_eps = 1e-6f;
        int64_t q_off = 0, k_off = 0, v_off = 0;        // columns of q, k, v in the stacked projection
    };
    // Short causal convolution + silu of the q, k, v channels of `proj` (history from the state), unit q and k heads:
    // [rows, 2 qk_heads dk + heads dv] fp32.  Then the state's history takes this step's last inputs.
    Tensor conv_silu_unit(const Tensor& proj, const Tensor& taps, const DeltaSpec& spec, const CacheView& view, const StepContext& ctx);
    // a_raw [rows, heads (* dk)], b_raw [rows, heads] (their row strides are used; one dtype), a_log [heads],
    // dt_bias [heads (* dk)]: beta = sigmoid(b_raw), decay = exp(-exp(a_log) * softplus(a_raw + dt_bias)); out [rows, heads * dv] fp32
    Tensor delta_scan(const Tensor& qkv, const Tensor& a_raw, const Tensor& b_raw, const Tensor& a_log, const Tensor& dt_bias,
                      const DeltaSpec& spec, const CacheView& view, const StepContext& ctx);

    // The generalized delta rule: S <- diag(w) S - (a u)(u^T S) + k v^T with both terms reading the old state, o = S^T r;
    // u = k / sqrt(sum k^2 + unit_eps) per head, w = exp(-rate * sigmoid(z + z_bias)), a = sigmoid(a_raw + a_bias).
    // proj [rows, >= ...] holds r, k (heads * dk each) and v (heads * dv) at the given columns; z, a_raw [rows, heads * dk] fp32;
    // view: a state of heads * dk * dv floats per sequence.  -> [rows, heads * dv] fp32
    struct GeneralDeltaSpec {
        int heads = 0, dk = 0, dv = 0;
        float rate = 1.f, unit_eps = 1e-6f;
        int64_t r_off = 0, k_off = 0, v_off = 0;
    };
    Tensor general_delta(const Tensor& proj, const Tensor& z, const Tensor& a_raw, const Tensor& z_bias, const Tensor& a_bias,
                         const GeneralDeltaSpec& spec, const CacheView& view, const StepContext& ctx);

    // ---- attention behind a window with pooled blocks, a sink, a query multiplier (csrc/attention_pooled.cu)
    struct PooledSpec {
        int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        int window = 0;                 // 0: every earlier token is seen
        int pool = 0;                   // > 0: blocks of this many tokens that lie wholly before the window are seen as one key and value
        float scale = 1.f;
        float temp_coef = 0.f;          // scores of the row at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
        int temp_every = 0;             // 0: no such multiplier
        const Tensor* sink = nullptr;   // [heads]: exp(sink_h) joins head h's denominator
        const Tensor* q_norm = nullptr; // [dim]: RMS norm of every query head with this weight (null: none)
        const Tensor* k_norm = nullptr;
        float eps = 1e-5f;
        const float* freq = nullptr;    // device [rot / 2]: pairs (i, i + rot / 2) of q and k turn by pos * freq[i]; null: no rotation
        float rot_mult = 1.f;
        int rot = 0;
        int64_t q_off = 0, k_off = 0, v_off = -1;       // columns of the stacked projection; v_off < 0: the values are the keys
    };
    // q (normed, rotated) goes back into proj; k (normed, rotated) and v go to the cache rows of the step's tokens; with
    // pooled blocks the blocks' sums (`pooled`: a view of 32-bit rows, one per `pool` positions) take the step's tokens
    void pooled_store(Tensor& proj, const PooledSpec& spec, const CacheView& tokens, const CacheView* pooled, const StepContext& ctx);
    // -> [rows, heads * vdim] in proj's dtype
    Tensor pooled_attention(const Tensor& proj, const PooledSpec& spec, const CacheView& tokens, const CacheView* pooled, const StepContext& ctx);

    // ---- attention over a cached latent (csrc/attention_latent.cu)
    struct LatentSpec {
        int heads = 0, dim = 0, rot = 0, rank = 0, vdim = 0;
        int rot_dims = 0;               // how many of the rot numbers turn (the first ones; 0: all)
        float scale = 1.f, eps = 1e-5f, rot_mult = 1.f;
        const float* freq = nullptr;    // device: rot / 2 angular frequencies
        int64_t q_off = 0, kv_off = 0, gate_off = -1;   // columns of the stacked projection: queries, [latent | key part], gates
    };
    // Interleaved rotary encoding in place: dims [first, first + dims) of each of `heads` heads (head_stride apart) of every row
    void rotate_pairs(Tensor& x, const StepContext& ctx, const float* freq, float mult, int heads, int64_t head_stride, int64_t first, int dims);
    // From a row of the stacked projection: [normed latent | rotated key part] in the activation dtype (what the cache keeps),
    // and the rotated query parts in their places of qf [rows, heads * (rank + rot)] fp32
    Tensor latent_prepare(const Tensor& proj, const Tensor& norm_w, const LatentSpec& spec, Tensor& qf, const StepContext& ctx);
    // out[row][h][n] = sum_k x[row][x_off + h * x_stride + k] * W_h: weights [heads * k, n] (per_head_rows_k) or [heads * n, k];
    // gate (null: none): the result is multiplied by sigmoid(gate[row][gate_off + h]); out: head h at h * out_stride
    void head_linear(const Tensor& x, int64_t x_off, int64_t x_stride, const Tensor& w, bool per_head_rows_k, Tensor& out,
                     int64_t out_stride, const Tensor* gate, int64_t gate_off, int heads, int k, int n, const StepContext& ctx);
    // Prompts in bfloat16: the same attention as products on the tensor cores, sequence by sequence and head by head, with keys
    // and values expanded from the gathered latents: scores = Q [Kn | R]^T (fp32), a masked softmax with the sink whose
    // weights are kept as two bf16 numbers each, result = [P_hi | P_lo] [V; V].  `proj` holds the queries with their rotated parts already
    // rotated; the step's rows are in the cache.  Returns [rows, heads * vdim] in proj's dtype, gates applied.
    Tensor latent_attention_prompt(const Tensor& proj, const Tensor& w_uk, const Tensor& w_uv, const Tensor* sink, const LatentSpec& spec,
                                   const CacheView& view, const StepContext& ctx);
    // qf [rows, heads * (rank + rot)] fp32 against the cached [latent | key part] rows -> [rows, heads * rank] fp32
    Tensor latent_attention(const Tensor& qf, const Tensor* sink, const LatentSpec& spec, const CacheView& view, const StepContext& ctx);

    // ---- routed experts (csrc/routed.cu)
    struct Routing {
        Tensor ids, weights, dense;     // [rows, top] int32, [rows, top] fp32, [rows, experts] fp32 (if asked for)
    };
    Routing route(const Tensor& logits, int top, bool softmax_all, bool with_dense);
    // scores sigmoid(logit); the choice runs on score + bias (null: none) among the experts of the `keep` best of `groups`
    // equally sized runs of adjacent experts (a group counts as the sum of its two largest); weights = score * scale of the chosen
    Routing route_scored(const Tensor& logits, int top, const Tensor* bias, int groups, int keep, float scale, bool with_dense);
    void scale_by_route(Tensor& act, const Tensor& dense, int experts, int inner);
    Tensor expert_gate_up(const Tensor& h, const Routing& r, const Tensor& w_gate_up, int top, int inner);
    Tensor expert_down_combine(const Tensor& act, const Routing& r, const Tensor& w_down, const Tensor& residual, int top, int inner);
    // Many rows: the rows are gathered expert by expert and every expert with rows runs its two products on the tensor
    // cores over its own rows only.  The host reads the experts' row counts (one small copy and a wait per call), so this
    // is for prompts, never inside a captured step.  w_gate_up [experts * 2 * inner, width] (gate and up row by row in
    // turn), w_down [width, experts * inner].
    Tensor experts_grouped(const Tensor& h, const Routing& r, const Tensor& w_gate_up, const Tensor& w_down, const Tensor& residual,
                           int top, int inner);

    // ---- matrix products: x [rows, k] @ weight [n, k]^T (+ bias [n]) (+ residual [rows, n])
    Tensor linear(const Rows& x, const Tensor& weight, const Tensor* bias = nullptr, const Tensor* residual = nullptr,
                  int out_dtype = -1, Tensor* out = nullptr);
    // linear(...) and the RMSNorm of its result.  For bf16 rows whose sizes allow it the norm is begun in the
    // product's epilogue and the second result is deferred; otherwise the norm's kernel runs.
    std::pair<Tensor, Rows> linear_norm(const Rows& x, const Tensor& weight, const Tensor& norm_weight, float eps,
                                        const Tensor* bias = nullptr, const Tensor* residual = nullptr);
    // linear(x, weight, bias) followed by rope_kv_write on its result; for up to 64 bf16 rows and a head size that
    // divides 128 both happen in the product's epilogue.
    Tensor qkv_rope_write(const Rows& x, const Tensor& weight, const Tensor* bias, const int* row_seq,
                          const int* row_pos, const float* denominators, int rotary_dim, int n_heads, int n_kv_heads,
                          int head_dim, const CacheView* view);
    // silu(x Wg^T) * (x Wu^T) for weight_pairs [2 * inner, k] whose rows alternate gate, up.
    // act 2: the tanh form of gelu instead of silu
    Tensor linear_swiglu(const Rows& x, const Tensor& weight_pairs, int act = 1);
    Tensor materialize(const Rows& h);

    // ---- attention of the step's rows over the paged cache.  q: the buffer that holds the queries, row stride
    // q_stride elements, head h at h * head_dim.
    // Values of another size than the keys (view.v_head_dim), first keys kept in sight behind a window
    // (view.keep_first) and a multiplier of the result run on the CUDA-core kernel.
    void attention(const Tensor& q, int64_t q_stride, Tensor& out, const CacheView& view, const StepContext& ctx,
                   int n_heads, int n_kv_heads, int head_dim, int window, float scale, float out_scale = 1.0f);

    // ---- attention whose heads' scores are mixed before the softmax (csrc/attention_talk.cu)
    struct TalkSpec {
        int heads = 0, kv_heads = 0, dim = 0, vdim = 0, window = 0;
        float scale = 1.f;
        const float* slopes = nullptr;  // device [heads]: slope_h * (i - j) is taken off head h's score; null: none
        const Tensor* talk = nullptr;   // [heads, heads]: score_h <- sum_g talk[h][g] score_g; null: none
        int64_t q_off = 0, k_off = 0, v_off = 0, gate_off = -1;     // columns of the stacked projection; gate_off < 0: no gate
    };
    // Keys and values of the step's rows go to the cache; blend (null: none) [rows, kv_heads * vdim] and lambda (one number):
    // v <- (1 - lambda) v + lambda blend first, and the blended values are what is kept; keep (null: none) receives the
    // values as stored
    void talk_store(Tensor& proj, const TalkSpec& spec, const CacheView& view, const StepContext& ctx, const Tensor* blend,
                    const Tensor* lambda, Tensor* keep);
    // -> [rows, heads * vdim] in proj's dtype: softmax over the window of the mixed scores, times the values, times
    // sigmoid(gate) element by element if the projection has gate columns
    Tensor talk_attention(const Tensor& proj, const TalkSpec& spec, const CacheView& view, const StepContext& ctx);

    // ---- sampling: one id per row of logits [rows, vocab] fp32
    void sample(const Tensor& logits, const float* temperature, const int* streams, const int* steps,
                unsigned long long seed, const int* row_live, int* out);

    // Raises KernelError if a kernel recorded that one of its bounded waits gave up (reads one word: call it
    // where the host waits for the device anyway); clears the word.
    void check_status();
    int* status_word() const { return (int*)status_.get(); }

    // ---- for tests and measurements
    Tensor linear_tc(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out,
                     int swap = -1, int bn = -1, int splits = -1, int act = 0, GemmFusion* fusion = nullptr);
    Tensor linear_simt(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out);
    bool tensor_core_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual) const;
    void plan(int64_t rows, int64_t n, int64_t k, bool* swapped, int* bn, int* splits = nullptr);
    int decode_splits(int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_kv_len);
    int attention_splits(int64_t rows, int n_heads, int max_kv_len) const;
    // FRIDAY_FUSE=0 keeps norms, rotation and cache write in kernels of their own (read at every call, for A/B runs)
    bool fusion_enabled() const;
    // For measurements: the next `launches` tensor-core products each fill one [sm_count][16] block of `trace`
    // (unsigned 64-bit) with their CTAs' time stamps (csrc/gemm_tc_fusion.h, part 4); null switches it off.
    void set_trace(unsigned long long* trace, int launches) { trace_ = trace; trace_left_ = launches; trace_next_ = 0; }
    long long launches() const { return launches_; }
    void add_launches(long long n) { launches_ += n; }

    // Event-bracketed time per kind of kernel (products, attention, everything else), switched on by
    // set_profile(true) or FRIDAY_PROFILE=1; read and cleared by take_profile (waits for the stream).
    enum Segment { Product = 0, Attention = 1, Other = 2, Segments = 3 };
    void set_profile(bool on);
    bool profiling() const { return profile_; }
    void take_profile(double ms[Segments], long long calls[Segments]);

private:
    struct Timed;
    friend struct Timed;
    bool few_rows_tile_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual,
                          int64_t max_rows, int columns = 128) const;
    void fusion_in(const Rows& x, GemmFusion& f) const;
    int device_, sms_;
    cudaStream_t stream_;
    DeviceBuffer tc_scratch_, tc_counters_, status_, attn_counters_;
    std::map<std::tuple<int64_t, int64_t, int64_t>, std::tuple<bool, int, int>> plans_;
    std::map<std::pair<int, int>, int> cluster_fit_;
    bool attn_tc_, profile_ = false;
    long long launches_ = 0;
    unsigned long long* trace_ = nullptr;
    int trace_left_ = 0, trace_next_ = 0;
    std::vector<std::tuple<int, cudaEvent_t, cudaEvent_t>> events_;
    std::vector<cudaEvent_t> spare_events_;
};

}  // namespace friday
