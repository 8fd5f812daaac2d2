// The operations of ops.h: which kernel runs for which shapes, and what is fused into what.
//
// The choices follow what was measured on a B200: a bf16 product goes to the tcgen05
// kernel whenever its operands' rows start on 16-byte boundaries and to the CUDA-core
// kernel otherwise (and always in float32: the true 32-bit path uses no tensor cores);
// one-token steps let norms, rotation and the cache write ride in the products'
// epilogues; prompts' attention runs both products on tcgen05, one-token steps split
// the keys over the CTAs of a cluster.
#include "friday/ops.h"

#include <stdlib.h>

#include <algorithm>
#include <string.h>

#include "ops/kernels.h"

namespace friday {

namespace {
inline int code(DType d) { return (int)d; }

bool env_on(const char* name, bool fallback = true) {
    const char* e = getenv(name);
    if (!e || !e[0]) return fallback;
    return e[0] != '0';
}

template <class K> void call(long long& launches, const K& k, int rc, const char* fn) {
    ++launches;
    if (rc != 0) throw KernelError(std::string(fn) + ": " + k.last_error());
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
}  // namespace

struct Ops::Timed {
    Ops& ops;
    cudaEvent_t a = nullptr, b = nullptr;
    int seg;
    Timed(Ops& o, int s) : ops(o), seg(s) {
        if (!ops.profile_) return;
        auto take = [&]() {
            cudaEvent_t e;
            if (!ops.spare_events_.empty()) { e = ops.spare_events_.back(); ops.spare_events_.pop_back(); }
            else cuda_check(cudaEventCreate(&e), "cudaEventCreate");
            return e;
        };
        a = take();
        b = take();
        cudaEventRecord(a, ops.stream_);
    }
    ~Timed() {
        if (!a) return;
        cudaEventRecord(b, ops.stream_);
        ops.events_.emplace_back(seg, a, b);
    }
};

Ops::Ops(int device, cudaStream_t stream) : device_(device), stream_(stream) {
    cuda_check(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    sms_ = prop.multiProcessorCount;
    // Partial tiles of split-k (at most two tiles of 128 x 256 floats per CTA, one CTA per SM), tile counters, and
    // the word in which a kernel records a wait that gave up: made once, so that captured graphs keep their addresses.
    tc_scratch_ = DeviceBuffer((size_t)2 * sms_ * 128 * 256 * sizeof(float));
    tc_counters_ = DeviceBuffer(4096 * sizeof(int), true);
    status_ = DeviceBuffer(4 * sizeof(int), true);
    attn_counters_ = DeviceBuffer(((size_t)1 << 16) * sizeof(int), true);
    attn_tc_ = env_on("FRIDAY_ATTN_TC");
    profile_ = env_on("FRIDAY_PROFILE", false);
}

Ops::~Ops() {
    for (auto& e : events_) { cudaEventDestroy(std::get<1>(e)); cudaEventDestroy(std::get<2>(e)); }
    for (auto e : spare_events_) cudaEventDestroy(e);
}

void Ops::set_profile(bool on) { profile_ = on; }

bool Ops::fusion_enabled() const { return env_on("FRIDAY_FUSE"); }

void Ops::take_profile(double ms[Segments], long long calls[Segments]) {
    for (int i = 0; i < Segments; ++i) { ms[i] = 0; calls[i] = 0; }
    if (events_.empty()) return;
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    for (auto& e : events_) {
        float t = 0;
        if (cudaEventElapsedTime(&t, std::get<1>(e), std::get<2>(e)) == cudaSuccess) {
            ms[std::get<0>(e)] += t;
            calls[std::get<0>(e)] += 1;
        }
        spare_events_.push_back(std::get<1>(e));
        spare_events_.push_back(std::get<2>(e));
    }
    events_.clear();
}

Tensor Ops::alloc(DType dtype, int64_t rows, int64_t cols) {
    if (!arena) throw KernelError("internal: an operation needs working memory and no arena is set");
    void* p = arena->alloc((size_t)rows * cols * dtype_size(dtype));
    return Tensor::make(p, dtype, {rows, cols});
}

float* Ops::scratch_floats(int64_t n) {
    if (!arena) throw KernelError("internal: an operation needs scratch memory and no arena is set");
    return (float*)arena->alloc((size_t)(n > 0 ? n : 1) * sizeof(float));
}

// ------------------------------------------------------------------ row-wise
Tensor Ops::embedding(const int* tokens, int64_t n, const Tensor& table, Tensor* out) {
    Tensor o = out ? *out : alloc(table.dtype, n, table.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.embedding(tokens, table.data, o.data, (int)n, (int)table.cols(), (int)table.rows(), code(table.dtype), stream_),
         "embedding");
    return o;
}

Tensor Ops::gather_rows(const int* rows, int64_t n, const Tensor& src) {
    if (!src.contiguous()) throw KernelError("gather_rows: the source must be contiguous");
    Tensor o = alloc(src.dtype, n, src.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.gather_rows(rows, src.data, o.data, (int)n, (int)src.cols(), code(src.dtype), stream_), "gather_rows");
    return o;
}

Tensor Ops::rmsnorm(const Tensor& x, const Tensor& weight, float eps, Tensor* out) {
    if (!x.contiguous() || weight.numel() != x.cols())
        throw KernelError(format("rmsnorm: rows of %lld columns (contiguous: %d), weight of %lld", (long long)x.cols(),
                                 (int)x.contiguous(), (long long)weight.numel()));
    Tensor o = out ? *out : alloc(x.dtype, x.rows(), x.cols());
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.rmsnorm(x.data, weight.data, code(weight.dtype), o.data, (int)x.rows(), (int)x.cols(), eps,
                                 code(x.dtype), stream_), "rmsnorm");
    return o;
}

Tensor Ops::swiglu(const Tensor& gate_up, int act) {
    if (!gate_up.contiguous() || gate_up.cols() % 2) throw KernelError("swiglu: rows must be contiguous pairs (gate, up)");
    const int64_t inner = gate_up.cols() / 2;
    Tensor o = alloc(gate_up.dtype, gate_up.rows(), inner);
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.gated_act(gate_up.data, o.data, (int)gate_up.rows(), (int)inner, act, code(gate_up.dtype), stream_), "gated_act");
    return o;
}

void Ops::rope_kv_write(Tensor& qkv, const int* row_seq, const int* row_pos, const float* denominators, int rotary_dim,
                        int n_heads, int n_kv_heads, int head_dim, const CacheView* view) {
    if (!qkv.contiguous() || qkv.cols() != (int64_t)(n_heads + 2 * n_kv_heads) * head_dim)
        throw KernelError("rope_kv_write: qkv must be contiguous rows of (heads + 2 kv heads) * head_dim");
    const bool write = view && view->write && view->k_pool;
    if (write && view->dtype != qkv.dtype) throw KernelError("rope_kv_write: the cache's dtype differs from the rows'");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k,
         k.rope_kv_write(qkv.data, row_seq, row_pos, denominators, denominators ? rotary_dim : 0, n_heads, n_kv_heads,
                         head_dim, write ? view->k_pool : nullptr, write ? view->v_pool : nullptr,
                         write ? view->block_table : nullptr, write ? view->table_width : 0,
                         view ? view->page_size : 0, write ? 1 : 0, (int)qkv.rows(), code(qkv.dtype), stream_),
         "rope_kv_write");
}

void Ops::advance(int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws, int n) {
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.advance(tokens, sampled, row_pos, kv_len, row_seq, draws, n, stream_), "advance");
}

void Ops::scale_rows(Tensor& x, float scale) {
    if (scale == 1.0f) return;
    if (!x.contiguous()) throw KernelError("scale_rows: rows must be contiguous");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.scale_rows(x.data, (long long)x.numel(), scale, code(x.dtype), stream_), "scale_rows");
}

void Ops::finish_logits(Tensor& logits, const Tensor* bias, float scale, float softcap) {
    if (!bias && scale == 1.0f && softcap <= 0.f) return;
    if (logits.dtype != DType::F32) throw KernelError("finish_logits: logits are float32");
    if (bias && bias->numel() != logits.cols()) throw KernelError("finish_logits: the bias does not match the vocabulary");
    const auto& k = kernels::rowwise();
    Timed t(*this, Other);
    call(launches_, k, k.finish_logits((float*)logits.data, (int)logits.rows(), (int)logits.cols(), (int)logits.ld,
                                       bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0, scale, softcap, stream_),
         "finish_logits");
}

// ------------------------------------------------------------------ a 32-bit residual stream
Tensor Ops::rmsnorm_to(const Tensor& x, const Tensor& weight, float offset, float eps, DType out_dtype) {
    if (!x.contiguous() || weight.numel() != x.cols())
        throw KernelError(format("rmsnorm: rows of %lld columns (contiguous: %d), weight of %lld", (long long)x.cols(),
                                 (int)x.contiguous(), (long long)weight.numel()));
    Tensor o = alloc(out_dtype, x.rows(), x.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.norm_cast(x.data, code(x.dtype), weight.data, code(weight.dtype), offset, o.data, code(out_dtype),
                                   (int)x.rows(), (int)x.cols(), eps, stream_), "norm_cast");
    return o;
}

Tensor Ops::concat_cast(const Tensor& a, const Tensor& b, DType out_dtype) {
    if (!a.contiguous() || !b.contiguous() || a.rows() != b.rows() || a.dtype != b.dtype)
        throw KernelError("concat_cast: two contiguous tensors of equal rows and dtype");
    Tensor o = alloc(out_dtype, a.rows(), a.cols() + b.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.concat_cast(a.data, b.data, code(a.dtype), o.data, code(out_dtype), (int)a.rows(), (int)a.cols(),
                                     (int)b.cols(), stream_), "concat_cast");
    return o;
}

Tensor Ops::add_scaled(const Tensor& residual, const Tensor& y, float alpha, const Tensor* z, float beta, bool in_place) {
    if (residual.dtype != DType::F32 || !residual.contiguous() || !y.contiguous() || y.numel() != residual.numel() ||
        (z && (z->dtype != y.dtype || !z->contiguous() || z->numel() != y.numel())))
        throw KernelError("add_scaled: a contiguous 32-bit residual and addends of its size");
    Tensor o = in_place ? residual : alloc(DType::F32, residual.rows(), residual.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.add_scaled((const float*)residual.data, y.data, alpha, z ? z->data : nullptr, beta, code(y.dtype),
                                    (float*)o.data, (long long)residual.numel(), stream_), "add_scaled");
    return o;
}

Tensor Ops::linear_residual(const Rows& x, const Tensor& weight, const Tensor* bias, const Tensor& residual, float alpha) {
    if (alpha == 1.0f && residual.dtype == x.t.dtype) return linear(x, weight, bias, &residual);
    if (residual.dtype != DType::F32) throw KernelError("linear_residual: a multiplier needs a 32-bit residual stream");
    // a 32-bit stream takes the product's 32-bit sums in the product's own epilogue where the rows are few (one kernel
    // less per product of a one-token step); for many rows the tensor-core product's 32-bit epilogue with a residual is its
    // slow one (measured on a 2,048-token prompt: 0.7 ms more in the products against 0.25 ms saved in the sums)
    if (alpha == 1.0f && (x.t.dtype == DType::F32 || x.t.rows() <= 128)) return linear(x, weight, bias, &residual, (int)DType::F32);
    Tensor y = linear(x, weight, bias, nullptr, (int)DType::F32);
    return add_scaled(residual, y, alpha);
}

Tensor Ops::layernorm_to(const Tensor& x, const Tensor& weight, const Tensor* bias, float eps, DType out_dtype) {
    if (!x.contiguous() || weight.numel() != x.cols() || (bias && (bias->numel() != x.cols() || bias->dtype != weight.dtype)))
        throw KernelError("layernorm: contiguous rows, a weight and a bias of their width and of one dtype");
    Tensor o = alloc(out_dtype, x.rows(), x.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.layernorm_cast(x.data, code(x.dtype), weight.data, bias ? bias->data : nullptr, code(weight.dtype), o.data,
                                        code(out_dtype), (int)x.rows(), (int)x.cols(), eps, stream_), "layernorm_cast");
    return o;
}

Tensor Ops::embed_rows(const int* tokens, int64_t n, const Tensor& table, float scale) {
    Tensor o = alloc(DType::F32, n, table.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.embed_rows(tokens, table.data, code(table.dtype), (float*)o.data, (int)n, (int)table.cols(), (int)table.rows(),
                                    scale, stream_), "embed_rows");
    return o;
}

Tensor Ops::embed_pos_rows(const StepContext& ctx, const Tensor& table, const Tensor& positions) {
    if (positions.cols() != table.cols() || positions.dtype != table.dtype || !positions.contiguous() || !table.contiguous())
        throw KernelError("embed_pos_rows: a token table and a position table of one width and dtype");
    Tensor o = alloc(DType::F32, ctx.rows, table.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.embed_pos(ctx.tokens, ctx.row_pos, table.data, positions.data, code(table.dtype), (float*)o.data, ctx.rows,
                                   (int)table.cols(), (int)table.rows(), (int)positions.rows(), stream_), "embed_pos");
    return o;
}

Tensor Ops::norm_shift(const Tensor& x, const Tensor& weight, float eps, const Tensor& shift, const CacheView& view, const StepContext& ctx,
                       DType out_dtype) {
    if (view.kind != CacheRequest::State || !view.state.defined()) throw KernelError("norm_shift needs a state view");
    if (x.dtype != DType::F32 || !x.contiguous() || weight.numel() != x.cols() || shift.numel() != x.cols())
        throw KernelError("norm_shift: a contiguous 32-bit stream, a weight and a shift of its width");
    Tensor o = alloc(out_dtype, x.rows(), x.cols());
    const long long stride = view.state.numel() / view.state.shape[0];
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.norm_shift((const float*)x.data, weight.data, code(weight.dtype), shift.data, code(shift.dtype), o.data,
                                    code(out_dtype), (float*)view.state.data, stride, ctx.row_seq, ctx.seq_start, ctx.seq_qlen,
                                    view.seq_slots, (int)x.rows(), ctx.n_seqs, (int)x.cols(), eps, ctx.decode ? 1 : 0, stream_),
         "norm_shift");
    if (!ctx.decode) ++launches_;
    return o;
}

Tensor Ops::post_norm_add(const Tensor& x, const Tensor& y, const Tensor& weight, float eps, float mult, const Tensor* next_weight,
                          float next_eps, DType next_dtype, Tensor* next) {
    if (x.dtype != DType::F32 || y.dtype != DType::F32 || !x.contiguous() || !y.contiguous() || x.numel() != y.numel() ||
        weight.numel() != x.cols() || (next_weight && (!next || next_weight->numel() != x.cols())))
        throw KernelError("post_norm_add: a contiguous 32-bit stream, a 32-bit addend of its size and weights of its width");
    Tensor o = alloc(DType::F32, x.rows(), x.cols());
    if (next_weight) *next = alloc(next_dtype, x.rows(), x.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.post_norm_add((const float*)x.data, (const float*)y.data, weight.data, code(weight.dtype), eps, mult,
                                       (float*)o.data, next_weight ? next_weight->data : nullptr, next_weight ? code(next_weight->dtype) : 0,
                                       next_eps, next_weight ? next->data : nullptr, code(next_dtype), (int)x.rows(), (int)x.cols(), stream_),
         "post_norm_add");
    return o;
}

void Ops::two_sided_act(Tensor& z, const Tensor& pq) {
    if (!z.contiguous() || pq.numel() != 2) throw KernelError("two_sided_act: contiguous rows and two numbers");
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.two_sided_act(z.data, (long long)z.numel(), code(z.dtype), pq.data, code(pq.dtype), stream_), "two_sided_act");
}

// ------------------------------------------------------------------ attention whose heads talk before the softmax
// FRIDAY_TALK_PROMPT=0 sends prompts through the CUDA-core kernels too (for comparisons)
static bool talk_prompt_allowed() {
    static const bool on = [] {
        const char* e = getenv("FRIDAY_TALK_PROMPT");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

void Ops::talk_store(Tensor& proj, const TalkSpec& s, const CacheView& view, const StepContext& ctx, const Tensor* blend,
                     const Tensor* lambda, Tensor* keep) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("talk_store needs a view of keys and values");
    if (view.dtype != proj.dtype) throw KernelError("talk_store: the cache's dtype differs from the rows'");
    const int64_t vw = (int64_t)s.kv_heads * s.vdim;
    if ((blend && (blend->dtype != proj.dtype || !blend->contiguous() || blend->rows() != proj.rows() || blend->cols() != vw || !lambda)) ||
        (keep && (keep->dtype != proj.dtype || !keep->contiguous() || keep->rows() != proj.rows() || keep->cols() != vw)))
        throw KernelError("talk_store: rows to blend with or to keep must be [rows, kv heads * value size] in the rows' dtype");
    if (!view.write && !keep) return;
    if (!view.write) throw KernelError("talk_store: a layer that leaves its values for others writes its own cache entry");
    const auto& k = kernels::attention_talk();
    Timed t(*this, Other);
    call(launches_, k, k.store(proj.data, (int)proj.ld, (int)s.k_off, (int)s.v_off, s.kv_heads, s.dim, s.vdim, ctx.row_seq, ctx.row_pos,
                               view.k_pool, view.v_pool, view.block_table, view.table_width, view.page_size, (int)proj.rows(),
                               code(proj.dtype), blend ? blend->data : nullptr, lambda ? lambda->data : nullptr,
                               lambda ? code(lambda->dtype) : 0, keep ? keep->data : nullptr, stream_), "talk_store");
}

Tensor Ops::talk_attention(const Tensor& proj, const TalkSpec& s, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("talk_attention needs a view of keys and values");
    if (view.dtype != proj.dtype) throw KernelError("talk_attention: the cache's dtype differs from the rows'");
    if (s.talk && (s.talk->numel() != (int64_t)s.heads * s.heads || !s.talk->contiguous()))
        throw KernelError("talk_attention: the mixing matrix is [heads, heads]");
    const auto& k = kernels::attention_talk();
    const int64_t rows = proj.rows();
    Tensor out = alloc(proj.dtype, rows, (int64_t)s.heads * s.vdim);
    const char* q = (const char*)proj.data + (size_t)s.q_off * dtype_size(proj.dtype);
    const char* gate = s.gate_off >= 0 ? (const char*)proj.data + (size_t)s.gate_off * dtype_size(proj.dtype) : nullptr;
    const size_t row_bytes = (size_t)proj.ld * dtype_size(proj.dtype);
    // Prompts in bfloat16 whose sizes the tensor-core kernels take: the mixed scores of all heads go through memory once
    // ([rows][heads][keys in sight] floats), the products run on the tensor cores.
    if (proj.dtype == DType::BF16 && !ctx.decode && ctx.n_seqs > 0 && ctx.rows == (int)rows && ctx.max_q_len >= 16 &&
        view.page_size == 64 && talk_prompt_allowed()) {
        const long long need = k.prompt_scratch_floats((int)rows, s.heads, s.dim, s.vdim, s.window, ctx.max_kv_len);
        const bool fits = need > 0 && need <= ((long long)1 << 29) && proj.ld % 8 == 0 && s.q_off % 8 == 0 && (s.gate_off < 0 || s.gate_off % 2 == 0);
        if (fits) {
            float* scratch = scratch_floats(need);
            Timed t(*this, Attention);
            call(launches_, k, k.prompt(q, (int)proj.ld, view.k_pool, view.v_pool, view.block_table, view.table_width, view.page_size,
                                        ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.n_seqs, (int)rows, ctx.max_q_len, s.heads, s.kv_heads,
                                        s.dim, s.vdim, s.window, ctx.max_kv_len, s.scale, s.slopes, s.talk ? s.talk->data : nullptr,
                                        s.talk ? code(s.talk->dtype) : 0, gate, (int)proj.ld, out.data, scratch, stream_), "talk_prompt");
            ++launches_;
            return out;
        }
    }
    // everything else: a row's keys in blocks, every block with all heads, then their merge; rows are taken in runs that
    // keep what the blocks leave below a gigabyte
    const int64_t per_row = std::max<int64_t>(1, k.scratch_floats(1, s.heads, s.vdim, s.window, ctx.max_kv_len));
    int64_t run = std::max<int64_t>(1, ((int64_t)1 << 28) / per_row);
    run = std::min(std::min(run, rows), (int64_t)65535);      // a row is a block index in y
    float* scratch = scratch_floats(run * per_row);
    for (int64_t r0 = 0; r0 < rows; r0 += run) {
        const int n = (int)std::min(run, rows - r0);
        Timed t(*this, Attention);
        call(launches_, k, k.rows(q + r0 * row_bytes, (int)proj.ld, view.k_pool, view.v_pool, view.block_table, view.table_width,
                                  view.page_size, ctx.row_seq + r0, ctx.row_pos + r0, n, s.heads, s.kv_heads, s.dim, s.vdim, s.window,
                                  ctx.max_kv_len, s.scale, s.slopes, s.talk ? s.talk->data : nullptr, s.talk ? code(s.talk->dtype) : 0,
                                  gate ? gate + r0 * row_bytes : nullptr, (int)proj.ld,
                                  (char*)out.data + (size_t)r0 * out.ld * dtype_size(out.dtype), scratch, code(proj.dtype), stream_),
             "talk_rows");
        ++launches_;
    }
    return out;
}

void Ops::kv_store(const Tensor& src, int64_t k_off, int64_t v_off, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("kv_store needs a view of keys and values");
    if (!view.write) return;
    if (view.dtype != src.dtype) throw KernelError("kv_store: the cache's dtype differs from the rows'");
    const int vd = view.v_head_dim > 0 ? view.v_head_dim : view.head_dim;
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.kv_store(src.data, (int)src.ld, (int)k_off, (int)v_off, view.n_kv_heads, view.head_dim, vd, ctx.row_seq,
                                  ctx.row_pos, view.k_pool, view.v_pool, view.block_table, view.table_width, view.page_size,
                                  (int)src.rows(), code(src.dtype), stream_), "kv_store");
}

void Ops::token_input(Tensor& x, const StepContext& ctx, const Tensor& table, int64_t col0, const Tensor& gate, const Tensor& proj,
                      const Tensor& norm, float eps) {
    const int64_t dim = gate.rows();
    if (x.dtype != DType::F32 || !x.contiguous()) throw KernelError("token_input: the residual stream must be contiguous 32-bit floats");
    if (gate.cols() != x.cols() || proj.rows() != x.cols() || proj.cols() != dim || norm.numel() != x.cols() ||
        col0 < 0 || col0 + dim > table.cols() || gate.dtype != table.dtype || proj.dtype != table.dtype)
        throw KernelError("token_input: gate [dim, width], proj [width, dim], norm [width] and a table slice of dim columns, one dtype");
    const auto& k = kernels::residual();
    if (x.rows() > 64 && table.dtype == DType::BF16 && dim % 8 == 0 && x.cols() % 8 == 0) {
        // many rows: both projections as products on the tensor cores (the stream rounded to bf16 for the first, as
        // for every other product), the steps between them row-wise
        Tensor xb = alloc(DType::BF16, x.rows(), x.cols());
        {
            Timed t(*this, Other);
            call(launches_, k, k.concat_cast(x.data, x.data, code(x.dtype), xb.data, code(DType::BF16), (int)x.rows(), (int)x.cols(), 0, stream_),
                 "concat_cast");
        }
        Tensor z = linear(Rows(xb), gate, nullptr, nullptr, (int)DType::F32);
        Tensor g = alloc(DType::BF16, x.rows(), dim);
        {
            Timed t(*this, Other);
            call(launches_, k, k.gelu_table((const float*)z.data, ctx.tokens, table.data, (int)table.ld, (int)col0, (int)table.rows(), g.data,
                                            (int)x.rows(), (int)dim, code(table.dtype), stream_), "gelu_table");
        }
        Tensor y = linear(Rows(g), proj, nullptr, nullptr, (int)DType::F32);
        Timed t(*this, Other);
        call(launches_, k, k.rms_add((float*)x.data, (const float*)y.data, norm.data, code(norm.dtype), (int)x.rows(), (int)x.cols(), eps, stream_),
             "rms_add");
        return;
    }
    float* g = scratch_floats(x.rows() * dim);
    Timed t(*this, Other);
    call(launches_, k, k.token_input((float*)x.data, ctx.tokens, ctx.row_seq, table.data, (int)table.ld, (int)col0, (int)table.rows(),
                                     gate.data, proj.data, norm.data, code(norm.dtype), (int)x.rows(), (int)x.cols(), (int)dim, eps, g,
                                     code(table.dtype), stream_), "token_input");
    ++launches_;
}

// ------------------------------------------------------------------ token pairs, the input convolution, two normed results
Tensor Ops::embed_pair_rows(const StepContext& ctx, const Tensor& table, const Tensor& pairs, int64_t buckets, int64_t mul_prev,
                            int64_t mul_cur, const CacheView& view) {
    if (view.kind != CacheRequest::State || view.state.dtype != DType::I32 || !view.seq_slots)
        throw KernelError("embed_pair_rows needs a state of one int32 per sequence");
    if (pairs.dtype != table.dtype || pairs.cols() != table.cols() || pairs.rows() != buckets + 1)
        throw KernelError("embed_pair_rows: the pair table has the token table's dtype and width and buckets + 1 rows");
    Tensor o = alloc(DType::F32, ctx.rows, table.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.embed_pair(ctx.tokens, ctx.row_seq, ctx.row_pos, ctx.seq_start, ctx.seq_qlen, view.seq_slots, table.data, pairs.data,
                                    code(table.dtype), (int*)view.state.data, (float*)o.data, ctx.rows, (int)table.cols(), (int)table.rows(),
                                    (int)buckets, (long long)mul_prev, (long long)mul_cur, stream_), "embed_pair");
    return o;
}

Tensor Ops::norm_conv(const Tensor& x, const Tensor& weight, const Tensor* bias, float eps, const Tensor& taps, const CacheView& view,
                      const StepContext& ctx, DType out_dtype) {
    const int64_t width = x.cols(), n = taps.cols();
    if (x.dtype != DType::F32 || !x.contiguous() || weight.numel() != width || (bias && (bias->numel() != width || bias->dtype != weight.dtype)) ||
        taps.rows() != width || !taps.contiguous())
        throw KernelError("norm_conv: a contiguous 32-bit stream, a weight (and bias) of its width, taps [width, n]");
    if (view.kind != CacheRequest::State || view.state.dtype != DType::F32 || view.state.numel() / view.state.shape[0] < (n - 1) * width)
        throw KernelError("norm_conv needs a state of (taps - 1) * width floats per sequence");
    const long long stride = view.state.numel() / view.state.shape[0];
    Tensor o = alloc(out_dtype, x.rows(), width);
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.norm_conv((const float*)x.data, weight.data, bias ? bias->data : nullptr, code(weight.dtype), taps.data, code(taps.dtype),
                                   (int)n, o.data, code(out_dtype), (float*)view.state.data, stride, 0, ctx.row_seq, ctx.seq_start, view.seq_slots,
                                   (int)x.rows(), (int)width, eps, ctx.decode ? 1 : 0, stream_), "norm_conv");
    if (!ctx.decode && n > 1)
        call(launches_, k, k.norm_conv_state((const float*)x.data, weight.data, bias ? bias->data : nullptr, code(weight.dtype), (int)n,
                                             code(out_dtype), (float*)view.state.data, stride, 0, ctx.seq_start, ctx.seq_qlen, view.seq_slots,
                                             ctx.n_seqs, (int)width, eps, stream_), "norm_conv_state");
    return o;
}

Tensor Ops::rms_pair_add(const Tensor& x, const Tensor& a, const Tensor& b, const Tensor& wa, const Tensor& wb, float eps, float mult) {
    if (x.dtype != DType::F32 || a.dtype != DType::F32 || b.dtype != DType::F32 || !x.contiguous() || !a.contiguous() || !b.contiguous() ||
        a.numel() != x.numel() || b.numel() != x.numel() || wa.numel() != x.cols() || wb.numel() != x.cols() || wa.dtype != wb.dtype)
        throw KernelError("rms_pair_add: a contiguous 32-bit stream, two 32-bit addends of its size, two weights of its width");
    Tensor o = alloc(DType::F32, x.rows(), x.cols());
    const auto& k = kernels::residual();
    Timed t(*this, Other);
    call(launches_, k, k.rms_pair_add((const float*)x.data, (const float*)a.data, (const float*)b.data, wa.data, wb.data, code(wa.dtype), eps, mult,
                                      (float*)o.data, (int)x.rows(), (int)x.cols(), stream_), "rms_pair_add");
    return o;
}

// ------------------------------------------------------------------ the generalized delta rule
Tensor Ops::general_delta(const Tensor& proj, const Tensor& z, const Tensor& a_raw, const Tensor& z_bias, const Tensor& a_bias,
                          const GeneralDeltaSpec& s, const CacheView& view, const StepContext& ctx) {
    const int64_t hk = (int64_t)s.heads * s.dk, hv = (int64_t)s.heads * s.dv;
    if (z.dtype != DType::F32 || a_raw.dtype != DType::F32 || z.cols() < hk || a_raw.cols() < hk || z_bias.numel() != hk || a_bias.numel() != hk ||
        z_bias.dtype != a_bias.dtype)
        throw KernelError("general_delta: 32-bit decay and removal projections of heads * dk columns, biases of that size and one dtype");
    if (view.kind != CacheRequest::State || view.state.dtype != DType::F32 || view.state.numel() / view.state.shape[0] < hk * s.dv)
        throw KernelError("general_delta needs a state of heads * dk * dv floats per sequence");
    const auto& k = kernels::delta();
    float* prep = scratch_floats(proj.rows() * hk * 5);
    Tensor o = alloc(DType::F32, proj.rows(), hv);
    Timed t(*this, Attention);                       // counted with the attention kernels and the other scans
    call(launches_, k, k.general_prepare(proj.data, (int)proj.ld, (int)s.r_off, (int)s.k_off, (const float*)z.data, (int)z.ld, (const float*)a_raw.data,
                                         (int)a_raw.ld, z_bias.data, a_bias.data, code(z_bias.dtype), prep, (int)proj.rows(), s.heads, s.dk, s.rate,
                                         s.unit_eps, code(proj.dtype), stream_), "general_prepare");
    call(launches_, k, k.general_scan(prep, proj.data, (int)proj.ld, (int)s.v_off, (float*)o.data, (float*)view.state.data,
                                      (long long)(view.state.numel() / view.state.shape[0]), 0, ctx.seq_start, ctx.seq_qlen, view.seq_slots, ctx.n_seqs,
                                      s.heads, s.dk, s.dv, code(proj.dtype), stream_), "general_scan");
    return o;
}

// ------------------------------------------------------------------ attention with pooled blocks, a sink, a query multiplier
static void check_pooled(const Ops::PooledSpec& s, const CacheView& tokens, const CacheView* pooled, DType dtype) {
    if (tokens.kind != CacheRequest::KV || !tokens.k_pool || tokens.dtype != dtype || tokens.n_kv_heads != s.kv_heads || tokens.head_dim != s.dim ||
        (tokens.v_head_dim > 0 ? tokens.v_head_dim : tokens.head_dim) != s.vdim || tokens.every != 1)
        throw KernelError("pooled attention: the cache view does not hold this mixer's keys and values in the rows' dtype");
    if ((s.pool > 0) != (pooled != nullptr)) throw KernelError("pooled attention: pooled blocks and their cache view go together");
    if (pooled && (pooled->kind != CacheRequest::KV || pooled->dtype != DType::F32 || pooled->every != s.pool || pooled->n_kv_heads != s.kv_heads ||
                   pooled->head_dim != s.dim || (pooled->v_head_dim > 0 ? pooled->v_head_dim : pooled->head_dim) != s.vdim))
        throw KernelError("pooled attention: the view of the pooled blocks must hold 32-bit rows of the keys' and values' sizes, one per block");
    if (s.v_off < 0 && (tokens.v_pool != tokens.k_pool || s.vdim != s.dim)) throw KernelError("pooled attention: values that are the keys share the keys' pool");
}

void Ops::pooled_store(Tensor& proj, const PooledSpec& s, const CacheView& tokens, const CacheView* pooled, const StepContext& ctx) {
    check_pooled(s, tokens, pooled, proj.dtype);
    const auto& k = kernels::attention_pooled();
    const int ndt = s.q_norm ? code(s.q_norm->dtype) : 0;
    if (s.q_norm && s.k_norm && s.q_norm->dtype != s.k_norm->dtype) throw KernelError("pooled attention: the two norm weights have one dtype");
    Timed t(*this, Other);
    call(launches_, k, k.prepare(proj.data, (int)proj.ld, (int)s.q_off, (int)s.k_off, (int)(s.v_off < 0 ? 0 : s.v_off), s.q_norm ? s.q_norm->data : nullptr,
                                 s.k_norm ? s.k_norm->data : nullptr, ndt, s.eps, s.freq, s.rot_mult, s.rot, tokens.k_pool,
                                 s.v_off < 0 ? nullptr : tokens.v_pool, tokens.block_table, tokens.table_width, tokens.page_size, ctx.row_seq,
                                 ctx.row_pos, (int)proj.rows(), s.heads, s.kv_heads, s.dim, s.vdim, tokens.write ? 1 : 0, code(proj.dtype), stream_),
         "pooled prepare");
    if (pooled && tokens.write)
        call(launches_, k, k.pool(tokens.k_pool, tokens.v_pool, (float*)pooled->k_pool, (float*)pooled->v_pool, tokens.block_table, tokens.table_width,
                                  pooled->block_table, pooled->table_width, tokens.page_size, ctx.seq_qlen, ctx.seq_pos0, ctx.n_seqs, ctx.max_q_len,
                                  s.kv_heads, s.dim, s.vdim, s.pool, code(proj.dtype), stream_), "pooled pool");
}

Tensor Ops::pooled_attention(const Tensor& proj, const PooledSpec& s, const CacheView& tokens, const CacheView* pooled, const StepContext& ctx) {
    check_pooled(s, tokens, pooled, proj.dtype);
    const auto& k = kernels::attention_pooled();
    Tensor out = alloc(proj.dtype, proj.rows(), (int64_t)s.heads * s.vdim);
    const float* pk = pooled ? (const float*)pooled->k_pool : nullptr;
    const float* pv = pooled ? (const float*)pooled->v_pool : nullptr;
    const int* ptable = pooled ? pooled->block_table : nullptr;
    const int pwidth = pooled ? pooled->table_width : 0;
    const bool tc = proj.dtype == DType::BF16 && !ctx.decode && ctx.max_q_len >= 16 && env_on("FRIDAY_POOLED_TC") &&
                    k.prompt_fits(s.dim, s.vdim, tokens.page_size) && ctx.n_seqs <= 65535;
    Timed t(*this, Attention);
    if (tc) {
        call(launches_, k, k.prompt(proj.data, (int)proj.ld, (int)s.q_off, out.data, tokens.k_pool, tokens.v_pool, pk, pv, tokens.block_table,
                                    tokens.table_width, ptable, pwidth, tokens.page_size, ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.n_seqs,
                                    ctx.max_q_len, s.heads, s.kv_heads, s.dim, s.vdim, s.window, s.pool, s.scale, s.temp_coef, s.temp_every,
                                    s.sink ? s.sink->data : nullptr, s.sink ? code(s.sink->dtype) : 0, stream_), "pooled prompt");
        return out;
    }
    // keys that a row can face: its window (or everything before it) and the pooled blocks
    int keys = ctx.max_kv_len;
    if (s.window > 0) keys = std::min(keys, s.window + (s.pool > 0 ? ctx.max_kv_len / s.pool : 0));
    const int splits = attention_splits(proj.rows(), s.heads, keys);
    float* scratch = scratch_floats(k.scratch_floats((int)proj.rows(), s.heads, s.vdim, splits));
    call(launches_, k, k.rows(proj.data, (int)proj.ld, (int)s.q_off, out.data, tokens.k_pool, tokens.v_pool, pk, pv, tokens.block_table,
                              tokens.table_width, ptable, pwidth, tokens.page_size, ctx.row_seq, ctx.row_pos, (int)proj.rows(), s.heads, s.kv_heads,
                              s.dim, s.vdim, s.window, s.pool, s.scale, s.temp_coef, s.temp_every, s.sink ? s.sink->data : nullptr,
                              s.sink ? code(s.sink->dtype) : 0, splits, scratch, code(proj.dtype), stream_), "pooled rows");
    ++launches_;                                     // the merge
    return out;
}

// ------------------------------------------------------------------ mixers with a matrix state
Tensor Ops::shift_mix(const Tensor& h, const std::vector<Tensor>& mu, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::State || !view.state.defined()) throw KernelError("shift_mix needs a state view");
    if (!h.contiguous() || mu.empty() || mu.size() > 8) throw KernelError("shift_mix: contiguous rows and 1 to 8 mixes");
    const void* ptrs[8] = {nullptr};
    for (size_t i = 0; i < mu.size(); ++i) {
        if (mu[i].numel() != h.cols() || mu[i].dtype != mu[0].dtype) throw KernelError("shift_mix: every mix is a vector of the width, one dtype");
        ptrs[i] = mu[i].data;
    }
    Tensor out = alloc(h.dtype, (int64_t)mu.size() * h.rows(), h.cols());
    const long long stride = view.state.numel() / view.state.shape[0];
    const auto& k = kernels::recurrence();
    Timed t(*this, Other);
    call(launches_, k, k.shift_mix(h.data, out.data, ptrs, (int)mu.size(), code(mu[0].dtype), (const float*)view.state.data, stride,
                                   ctx.row_seq, ctx.seq_start, view.seq_slots, (int)h.rows(), (int)h.cols(), code(h.dtype), stream_),
         "shift_mix");
    return out;
}

void Ops::tanh_rows(Tensor& x) {
    if (!x.contiguous()) throw KernelError("tanh_rows: rows must be contiguous");
    const auto& k = kernels::recurrence();
    Timed t(*this, Other);
    call(launches_, k, k.tanh_rows(x.data, (long long)x.numel(), code(x.dtype), stream_), "tanh_rows");
}

Tensor Ops::state_scan(const Tensor& q, const Tensor& kk, const Tensor& v, const Tensor& z, const ScanSpec& s, const CacheView& view,
                       const StepContext& ctx) {
    if (view.kind != CacheRequest::State || !view.state.defined() || view.state.dtype != DType::F32)
        throw KernelError("state_scan needs a 32-bit state view");
    if (q.dtype != kk.dtype || q.dtype != v.dtype || z.dtype != DType::F32 || !z.contiguous() || z.cols() != (int64_t)s.heads * s.dk)
        throw KernelError("state_scan: q, k, v of one dtype and fp32 decays [rows, heads * dk]");
    const long long stride = view.state.numel() / view.state.shape[0];
    if (s.state_offset + (long long)s.heads * s.dk * s.dv > stride) throw KernelError("state_scan: the state is smaller than the heads' matrices");
    Tensor out = alloc(DType::F32, q.rows(), (int64_t)s.heads * s.dv);
    const auto& k = kernels::recurrence();
    long long seg_floats = 0;
    const int seg_len = k.scan_plan(ctx.n_seqs, ctx.max_q_len, s.heads, s.dk, s.dv, &seg_floats);
    float* seg_scratch = seg_len > 0 ? scratch_floats(seg_floats) : nullptr;
    Timed t(*this, Attention);
    call(launches_, k,
         k.scan(q.data, (int)q.ld, kk.data, (int)kk.ld, v.data, (int)v.ld, (const float*)z.data, s.z_bias ? s.z_bias->data : nullptr,
                s.z_bias ? code(s.z_bias->dtype) : 0, s.bonus ? s.bonus->data : nullptr, s.bonus ? code(s.bonus->dtype) : 0,
                (float*)out.data, (float*)view.state.data, stride, (long long)s.state_offset, s.carry ? s.carry->data : nullptr,
                s.carry ? (int)s.carry->cols() : 0, ctx.row_seq, ctx.seq_start, ctx.seq_qlen, view.seq_slots, ctx.n_seqs,
                ctx.max_q_len, s.heads, s.dk, s.dv, s.mode, s.q_scale, s.tau, seg_len, seg_scratch, code(q.dtype), stream_),
         "scan");
    return out;
}

Tensor Ops::head_norm_gate(const Tensor& o, const Tensor& gate, const Tensor& weight, bool weight_per_head, int heads, int dv,
                           float eps, float out_scale, DType dtype, const StepContext& ctx, bool gate_sigmoid) {
    if (o.dtype != DType::F32 || !o.contiguous() || o.cols() != (int64_t)heads * dv || gate.dtype != dtype ||
        weight.numel() != (weight_per_head ? (int64_t)heads * dv : (int64_t)dv))
        throw KernelError("head_norm_gate: fp32 rows [rows, heads * dv], a gate in the result's dtype, a weight per channel");
    Tensor out = alloc(dtype, o.rows(), o.cols());
    const auto& k = kernels::recurrence();
    Timed t(*this, Other);
    call(launches_, k, k.head_norm_gate((const float*)o.data, gate.data, (int)gate.ld, out.data, weight.data, code(weight.dtype),
                                        weight_per_head ? 1 : 0, ctx.row_seq, (int)o.rows(), heads, dv, eps, out_scale,
                                        gate_sigmoid ? 1 : 0, code(dtype), stream_), "head_norm_gate");
    return out;
}

// ------------------------------------------------------------------ the delta rule
Tensor Ops::conv_silu_unit(const Tensor& proj, const Tensor& taps, const DeltaSpec& s, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::State || !view.state.defined() || view.state.dtype != DType::F32)
        throw KernelError("conv_silu_unit needs a 32-bit state view");
    const int64_t qk = (int64_t)s.qk_heads * s.dk, channels = 2 * qk + (int64_t)s.heads * s.dv;
    const long long stride = view.state.numel() / view.state.shape[0];
    if (taps.numel() != channels * s.taps || (int64_t)(s.taps - 1) * channels + (int64_t)s.heads * s.dk * s.dv > stride)
        throw KernelError("conv_silu_unit: taps [channels, taps] and a state that holds taps - 1 rows of inputs before the heads' matrices");
    Tensor out = alloc(DType::F32, proj.rows(), channels);
    const auto& k = kernels::delta();
    Timed t(*this, Other);
    call(launches_, k, k.conv_prepare(proj.data, (int)proj.ld, (int)s.q_off, (int)s.k_off, (int)s.v_off, taps.data, code(taps.dtype),
                                      (float*)out.data, (const float*)view.state.data, stride, ctx.row_seq, ctx.seq_start, view.seq_slots,
                                      (int)proj.rows(), s.qk_heads, s.dk, s.heads * s.dv, s.taps, s.q_scale, s.unit_eps, ctx.decode ? 1 : 0,
                                      code(proj.dtype), stream_), "conv_prepare");
    if (s.taps > 1 && !ctx.decode)
        call(launches_, k, k.conv_state(proj.data, (int)proj.ld, (int)s.q_off, (int)s.k_off, (int)s.v_off, (float*)view.state.data, stride,
                                        ctx.row_seq, ctx.seq_start, ctx.seq_qlen, view.seq_slots, ctx.n_seqs, s.qk_heads, s.dk,
                                        s.heads * s.dv, s.taps, code(proj.dtype), stream_), "conv_state");
    return out;
}

Tensor Ops::delta_scan(const Tensor& qkv, const Tensor& a_raw, const Tensor& b_raw, const Tensor& a_log, const Tensor& dt_bias,
                       const DeltaSpec& s, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::State || !view.state.defined() || view.state.dtype != DType::F32)
        throw KernelError("delta_scan needs a 32-bit state view");
    const int64_t channels = 2 * (int64_t)s.qk_heads * s.dk + (int64_t)s.heads * s.dv;
    if (qkv.dtype != DType::F32 || !qkv.contiguous() || qkv.cols() != channels || a_raw.dtype != b_raw.dtype ||
        a_log.numel() != s.heads || a_log.dtype != dt_bias.dtype || dt_bias.numel() != (s.per_channel ? (int64_t)s.heads * s.dk : (int64_t)s.heads))
        throw KernelError("delta_scan: fp32 q, k, v rows, raw decays and betas of one dtype, a rate per head and a bias per decay");
    const long long stride = view.state.numel() / view.state.shape[0];
    const long long s_off = (long long)(s.taps - 1) * channels;
    Tensor out = alloc(DType::F32, qkv.rows(), (int64_t)s.heads * s.dv);
    const auto& k = kernels::delta();
    Timed t(*this, Attention);
    call(launches_, k, k.scan((const float*)qkv.data, a_raw.data, (int)a_raw.ld, b_raw.data, (int)b_raw.ld, code(a_raw.dtype), a_log.data,
                              dt_bias.data, code(a_log.dtype), (float*)out.data, (float*)view.state.data, stride, s_off, ctx.row_seq,
                              ctx.seq_start, ctx.seq_qlen, view.seq_slots, ctx.n_seqs, s.heads, s.qk_heads, s.dk, s.dv,
                              s.per_channel ? 1 : 0, stream_), "delta_scan");
    return out;
}

// ------------------------------------------------------------------ attention over a cached latent
void Ops::rotate_pairs(Tensor& x, const StepContext& ctx, const float* freq, float mult, int heads, int64_t head_stride, int64_t first,
                       int dims) {
    const auto& k = kernels::attention_latent();
    Timed t(*this, Other);
    call(launches_, k, k.rotate_pairs(x.data, (int)x.ld, ctx.row_seq, ctx.row_pos, freq, mult, (int)x.rows(), heads, (int)head_stride,
                                      (int)first, dims, code(x.dtype), stream_), "rotate_pairs");
}

Tensor Ops::latent_prepare(const Tensor& proj, const Tensor& norm_w, const LatentSpec& s, Tensor& qf, const StepContext& ctx) {
    if (qf.dtype != DType::F32 || !qf.contiguous() || qf.cols() != (int64_t)s.heads * (s.rank + s.rot) || norm_w.numel() != s.rank)
        throw KernelError("latent_prepare: fp32 queries [rows, heads * (rank + rot)] and a norm weight of the latent's size");
    Tensor ckr = alloc(proj.dtype, proj.rows(), (int64_t)s.rank + s.rot);
    const auto& k = kernels::attention_latent();
    Timed t(*this, Other);
    call(launches_, k, k.prepare(proj.data, (int)proj.ld, (int)s.q_off, (int)s.kv_off, ckr.data, (float*)qf.data, norm_w.data,
                                 code(norm_w.dtype), s.eps, ctx.row_seq, ctx.row_pos, s.freq, s.rot_mult, (int)proj.rows(), s.heads, s.dim,
                                 s.rot, s.rot_dims > 0 ? s.rot_dims : s.rot, s.rank, code(proj.dtype), stream_), "latent_prepare");
    return ckr;
}

void Ops::head_linear(const Tensor& x, int64_t x_off, int64_t x_stride, const Tensor& w, bool per_head_rows_k, Tensor& out,
                      int64_t out_stride, const Tensor* gate, int64_t gate_off, int heads, int k_, int n, const StepContext& ctx) {
    if (!w.contiguous() || w.numel() != (int64_t)heads * k_ * n || (gate && gate->dtype != out.dtype))
        throw KernelError("head_linear: contiguous weights of heads * k * n numbers, a gate in the result's dtype");
    const auto& k = kernels::attention_latent();
    Timed t(*this, Product);
    call(launches_, k, k.head_linear(x.data, code(x.dtype), (int)x.ld, (int)x_off, (int)x_stride, w.data, code(w.dtype),
                                     per_head_rows_k ? 0 : 1, out.data, code(out.dtype), (int)out.ld, (int)out_stride,
                                     gate ? gate->data : nullptr, gate ? (int)gate->ld : 0, (int)gate_off, ctx.row_seq, (int)x.rows(),
                                     heads, k_, n, stream_), "head_linear");
}

Tensor Ops::latent_attention(const Tensor& qf, const Tensor* sink, const LatentSpec& s, const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("latent_attention needs a view of cached rows");
    const int vd = view.v_head_dim > 0 ? view.v_head_dim : view.head_dim;
    if (view.n_kv_heads != 1 || view.head_dim != s.rank || vd != s.rot || (sink && sink->numel() != s.heads))
        throw KernelError("latent_attention: the cache keeps one row [latent | key part] per position, the sink one number per head");
    const int rows = (int)qf.rows();
    Tensor out = alloc(DType::F32, rows, (int64_t)s.heads * s.rank);
    const int splits = attention_splits(rows, s.heads, ctx.max_kv_len);
    float* scratch = splits > 1 ? scratch_floats((int64_t)rows * s.heads * splits * (s.rank + 2)) : nullptr;
    const auto& k = kernels::attention_latent();
    Timed t(*this, Attention);
    call(launches_, k, k.run((const float*)qf.data, (float*)out.data, view.k_pool, view.v_pool, view.block_table, view.table_width,
                             view.page_size, ctx.row_seq, ctx.row_pos, sink ? sink->data : nullptr, sink ? code(sink->dtype) : 0, rows,
                             s.heads, s.rank, s.rot, s.scale, splits, scratch, code(view.dtype), stream_), "attention_latent");
    if (splits > 1) ++launches_;
    return out;
}

Tensor Ops::latent_attention_prompt(const Tensor& proj, const Tensor& w_uk, const Tensor& w_uv, const Tensor* sink, const LatentSpec& s,
                                    const CacheView& view, const StepContext& ctx) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("latent_attention needs a view of cached rows");
    if (proj.dtype != DType::BF16 || view.dtype != DType::BF16 || (int)ctx.q_lens.size() != ctx.n_seqs || (int)ctx.kv_lens.size() != ctx.n_seqs)
        throw KernelError("latent_attention_prompt: bfloat16 rows and a step whose lengths the host knows");
    const auto& k = kernels::attention_latent();
    const int64_t hv = (int64_t)s.heads * s.vdim;
    Tensor of = alloc(DType::F32, proj.rows(), hv);
    int64_t r0 = 0;
    for (int q = 0; q < ctx.n_seqs; ++q) {
        const int64_t T = ctx.q_lens[(size_t)q], n = ctx.kv_lens[(size_t)q], n_pad = (n + 7) / 8 * 8;
        if (T <= 0) continue;
        Tensor c_all = alloc(DType::BF16, 2 * n_pad, s.rank), r_all = alloc(DType::BF16, n_pad, s.rot);
        {
            Timed t(*this, Attention);
            call(launches_, k, k.gather(view.k_pool, view.v_pool, view.block_table + (size_t)q * view.table_width, view.page_size, (int)n,
                                        (int)n_pad, s.rank, s.rot, c_all.data, r_all.data, code(DType::BF16), stream_), "latent gather");
        }
        const int64_t hd = (int64_t)s.dim + s.rot;
        Tensor kn = linear(Rows(c_all.row_slice(0, n_pad)), w_uk);      // [n_pad, heads * dim]: every head's unrotated keys
        Tensor kcat = alloc(DType::BF16, n_pad, s.heads * hd);          // [n_pad, heads, dim + rot]: whole keys, head by head
        {
            Timed t(*this, Attention);
            call(launches_, k, k.key_concat(kn.data, r_all.data, (int)n_pad, s.heads, s.dim, s.rot, kcat.data, code(DType::BF16), stream_),
                 "key_concat");
        }
        Tensor vt = linear(Rows(w_uv), c_all);                          // [heads * vdim, 2 n_pad]: values, transposed, twice side by side
        Tensor scores = alloc(DType::F32, T, n_pad);
        Tensor weights = alloc(DType::BF16, T, 2 * n_pad);              // every weight as two bf16 numbers: [hi | lo]
        const Tensor rows = proj.row_slice(r0, T);
        for (int h = 0; h < s.heads; ++h) {
            Tensor qh = rows, kh = kcat, vh = vt.row_slice((int64_t)h * s.vdim, s.vdim);
            qh.data = (char*)rows.data + (size_t)(s.q_off + (int64_t)h * hd) * 2;
            qh.shape[1] = hd;
            kh.data = (char*)kcat.data + (size_t)h * hd * 2;
            kh.shape[1] = hd;
            linear(Rows(qh), kh, nullptr, nullptr, (int)DType::F32, &scores);
            {
                Timed t(*this, Attention);
                call(launches_, k, k.softmax_split((const float*)scores.data, (int)scores.ld, (int)T, (int)n_pad, (int)(n - T), s.scale,
                                                   sink ? sink->data : nullptr, sink ? code(sink->dtype) : 0, h, weights.data,
                                                   (char*)weights.data + (size_t)n_pad * 2, (int)(2 * n_pad), stream_), "softmax_split");
            }
            Tensor oh = of.row_slice(r0, T);
            oh.data = (char*)oh.data + (size_t)h * s.vdim * 4;
            oh.shape[1] = s.vdim;
            linear(Rows(weights), vh, nullptr, nullptr, (int)DType::F32, &oh);
        }
        r0 += T;
    }
    Tensor out = alloc(proj.dtype, proj.rows(), hv);
    Timed t(*this, Other);
    call(launches_, k, k.gate_cast((const float*)of.data, s.gate_off >= 0 ? proj.data : nullptr, (int)proj.ld, (int)s.gate_off,
                                   (int)proj.rows(), s.heads, s.vdim, out.data, code(proj.dtype), stream_), "gate_cast");
    return out;
}

// ------------------------------------------------------------------ routed experts
Ops::Routing Ops::route(const Tensor& logits, int top, bool softmax_all, bool with_dense) {
    if (logits.dtype != DType::F32) throw KernelError("route: router logits are float32");
    Routing r;
    const int64_t rows = logits.rows(), experts = logits.cols();
    r.ids = Tensor::make(arena->alloc((size_t)rows * top * sizeof(int)), DType::I32, {rows, (int64_t)top});
    r.weights = alloc(DType::F32, rows, top);
    if (with_dense) r.dense = alloc(DType::F32, rows, experts);
    const auto& k = kernels::routed();
    Timed t(*this, Other);
    call(launches_, k, k.route((const float*)logits.data, (int)logits.ld, (int)rows, (int)experts, top, softmax_all ? 1 : 0,
                               (int*)r.ids.data, (float*)r.weights.data, with_dense ? (float*)r.dense.data : nullptr, stream_), "route");
    return r;
}

Ops::Routing Ops::route_scored(const Tensor& logits, int top, const Tensor* bias, int groups, int keep, float scale, bool with_dense) {
    if (logits.dtype != DType::F32) throw KernelError("route: router logits are float32");
    const int64_t rows = logits.rows(), experts = logits.cols();
    if (bias && bias->numel() != experts) throw KernelError("route: the choice bias has a number per expert");
    Routing r;
    r.ids = Tensor::make(arena->alloc((size_t)rows * top * sizeof(int)), DType::I32, {rows, (int64_t)top});
    r.weights = alloc(DType::F32, rows, top);
    if (with_dense) r.dense = alloc(DType::F32, rows, experts);
    const auto& k = kernels::routed();
    Timed t(*this, Other);
    call(launches_, k, k.route_scored((const float*)logits.data, (int)logits.ld, (int)rows, (int)experts, top, bias ? bias->data : nullptr,
                                      bias ? code(bias->dtype) : 0, groups, keep, scale, (int*)r.ids.data, (float*)r.weights.data,
                                      with_dense ? (float*)r.dense.data : nullptr, stream_), "route_scored");
    return r;
}

void Ops::scale_by_route(Tensor& act, const Tensor& dense, int experts, int inner) {
    if (!act.contiguous() || act.cols() != (int64_t)experts * inner || dense.rows() != act.rows()) throw KernelError("scale_by_route: shapes");
    const auto& k = kernels::routed();
    Timed t(*this, Other);
    call(launches_, k, k.scale_by_route(act.data, (const float*)dense.data, (int)act.rows(), experts, inner, code(act.dtype), stream_),
         "scale_by_route");
}

Tensor Ops::expert_gate_up(const Tensor& h, const Routing& r, const Tensor& w_gate_up, int top, int inner) {
    if (!h.contiguous() || h.dtype != w_gate_up.dtype || !w_gate_up.contiguous() || w_gate_up.cols() != h.cols())
        throw KernelError("expert_gate_up: rows and stacked gate/up weights of one dtype and width");
    Tensor act = alloc(h.dtype, h.rows() * top, inner);
    const auto& k = kernels::routed();
    Timed t(*this, Product);
    call(launches_, k, k.gate_up(h.data, (const int*)r.ids.data, w_gate_up.data, act.data, (int)h.rows(), top,
                                 (int)(w_gate_up.rows() / (2 * (int64_t)inner)), (int)h.cols(), inner, code(h.dtype), stream_), "gate_up");
    return act;
}

Tensor Ops::expert_down_combine(const Tensor& act, const Routing& r, const Tensor& w_down, const Tensor& residual, int top, int inner) {
    if (act.dtype != w_down.dtype) throw KernelError("expert_down_combine: activations and weights of one dtype");
    Tensor out = alloc(residual.dtype, residual.rows(), residual.cols());
    const auto& k = kernels::routed();
    const long long need = k.down_scratch_floats((int)residual.rows(), top, (int)residual.cols(), inner, code(act.dtype));
    float* scratch = need > 0 ? scratch_floats(need) : nullptr;
    Timed t(*this, Product);
    call(launches_, k, k.down_combine(act.data, (const int*)r.ids.data, (const float*)r.weights.data, w_down.data, (int)w_down.ld,
                                      residual.data, out.data, code(residual.dtype), (int)residual.rows(), top,
                                      (int)(w_down.cols() / inner), (int)residual.cols(), inner, scratch, code(act.dtype), stream_),
         "down_combine");
    if (need > 0) ++launches_;
    return out;
}

Tensor Ops::experts_grouped(const Tensor& h, const Routing& r, const Tensor& w_gate_up, const Tensor& w_down, const Tensor& residual,
                            int top, int inner) {
    const int64_t rows = h.rows(), width = h.cols(), n_pairs = rows * top;
    const int experts = (int)(w_gate_up.rows() / (2 * (int64_t)inner));
    const auto& k = kernels::routed();
    int* offsets = (int*)arena->alloc((size_t)(experts + 1) * sizeof(int));
    int* pos = (int*)arena->alloc((size_t)n_pairs * sizeof(int));
    int* row_at = (int*)arena->alloc((size_t)n_pairs * sizeof(int));
    {
        Timed t(*this, Other);
        call(launches_, k, k.sort_pairs((const int*)r.ids.data, (int)rows, top, experts, offsets, pos, row_at, stream_), "sort_pairs");
    }
    std::vector<int> off((size_t)experts + 1);
    cuda_check(cudaMemcpyAsync(off.data(), offsets, off.size() * sizeof(int), cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    Tensor gathered = gather_rows(row_at, n_pairs, h);
    Tensor part = alloc(DType::F32, n_pairs, width);
    for (int e = 0; e < experts; ++e) {
        const int64_t lo = off[(size_t)e], n = off[(size_t)e + 1] - lo;
        if (n <= 0) continue;
        Tensor act = linear_swiglu(Rows(gathered.row_slice(lo, n)), w_gate_up.row_slice((int64_t)e * 2 * inner, 2 * (int64_t)inner));
        Tensor wd = w_down;                          // this expert's columns, the matrix's row stride
        wd.data = (char*)w_down.data + (size_t)e * inner * dtype_size(w_down.dtype);
        wd.shape[1] = inner;
        Tensor out = part.row_slice(lo, n);
        linear(Rows(act), wd, nullptr, nullptr, (int)DType::F32, &out);
    }
    Tensor result = alloc(residual.dtype, residual.rows(), residual.cols());
    Timed t(*this, Other);
    call(launches_, k, k.combine((const float*)part.data, (const int*)r.ids.data, (const float*)r.weights.data, pos, residual.data,
                                 result.data, code(residual.dtype), (int)rows, top, (int)width, stream_), "combine");
    return result;
}

// ------------------------------------------------------------------ matrix products
bool Ops::tensor_core_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual) const {
    (void)residual;
    return x.dtype == DType::BF16 && weight.dtype == DType::BF16 && (out.dtype == DType::BF16 || out.dtype == DType::F32) &&
           x.cols() % 8 == 0 && x.ld % 8 == 0 && weight.ld % 8 == 0 && aligned16(x.data) && aligned16(weight.data);
}

bool Ops::few_rows_tile_ok(const Tensor& x, const Tensor& weight, const Tensor& out, const Tensor* residual,
                           int64_t max_rows, int columns) const {
    return fusion_enabled() && out.dtype == DType::BF16 && x.rows() <= max_rows && weight.rows() % columns == 0 && out.ld % 8 == 0 &&
           aligned16(out.data) && (!residual || aligned16(residual->data)) && tensor_core_ok(x, weight, out, residual);
}

void Ops::fusion_in(const Rows& x, GemmFusion& f) const {
    if (!x.deferred) return;
    f.in_ssq = (const float*)x.ssq.data;
    f.in_parts = (int)x.ssq.rows();
    f.in_width = (float)x.t.cols();
    f.in_eps = x.eps;
}

void Ops::plan(int64_t rows, int64_t n, int64_t k, bool* swapped, int* bn, int* splits) {
    auto key = std::make_tuple(rows, n, k);
    auto it = plans_.find(key);
    if (it == plans_.end()) {
        long long p[8] = {0};
        const auto& g = kernels::gemm_tc();
        if (g.plan((int)rows, (int)n, (int)k, sms_, -1, -1, -1, p) != 0)
            throw KernelError(std::string("gemm_tc_plan: ") + g.last_error());
        if (plans_.size() > 4096) plans_.clear();
        it = plans_.emplace(key, std::make_tuple(p[0] != 0, (int)p[1], (int)p[2])).first;
    }
    if (swapped) *swapped = std::get<0>(it->second);
    if (bn) *bn = std::get<1>(it->second);
    if (splits) *splits = std::get<2>(it->second);
}

static void check_residual(const Tensor* residual, const Tensor& out) {
    if (!residual) return;
    if (residual->rows() != out.rows() || residual->cols() != out.cols() || residual->dtype != out.dtype ||
        residual->ld != out.ld)
        throw KernelError("linear: the residual must have the result's shape, dtype and row stride");
}

Tensor Ops::linear_tc(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out,
                      int swap, int bn, int splits, int act, GemmFusion* fusion) {
    const auto& g = kernels::gemm_tc();
    Timed t(*this, Product);
    GemmFusion traced;
    if (trace_ && trace_next_ < trace_left_) {
        if (fusion) traced = *fusion;
        else memset(&traced, 0, sizeof traced);
        traced.trace = trace_ + (size_t)trace_next_++ * sms_ * 16;
        fusion = &traced;
    }
    call(launches_, g,
         g.fused(x.data, weight.data, out.data, code(out.dtype), bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0,
                 residual ? residual->data : nullptr, (int)x.rows(), (int)weight.rows(), (int)x.cols(), (int)x.ld,
                 (int)weight.ld, (int)out.ld, (float*)tc_scratch_.get(), (long long)(tc_scratch_.bytes() / sizeof(float)),
                 (int*)tc_counters_.get(), (int)(tc_counters_.bytes() / sizeof(int)), (int*)status_.get(), sms_, swap, bn,
                 splits, act, fusion, stream_),
         "gemm_tc_fused");
    return out;
}

Tensor Ops::linear_simt(const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, Tensor& out) {
    const auto& g = kernels::gemm_simt();
    Timed t(*this, Product);
    call(launches_, g,
         g.gemm(x.data, code(x.dtype), weight.data, code(weight.dtype), out.data, code(out.dtype),
                bias ? bias->data : nullptr, bias ? code(bias->dtype) : 0, residual ? residual->data : nullptr,
                (int)x.rows(), (int)weight.rows(), (int)x.cols(), (int)x.ld, (int)weight.ld, (int)out.ld, stream_),
         "gemm_simt");
    return out;
}

static void check_product(const Tensor& x, const Tensor& weight) {
    if (x.ndim != 2 || weight.ndim != 2)
        throw KernelError("linear: input and weight must be 2-d");
    if (weight.cols() != x.cols())
        throw KernelError(format("linear: input has %lld columns, weight is [%lld, %lld]", (long long)x.cols(),
                                 (long long)weight.rows(), (long long)weight.cols()));
}

Tensor Ops::linear(const Rows& x, const Tensor& weight, const Tensor* bias, const Tensor* residual, int out_dtype,
                   Tensor* out) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const DType od = out_dtype < 0 ? xt.dtype : (DType)out_dtype;
    Tensor o = out ? *out : alloc(od, xt.rows(), weight.rows());
    check_residual(residual, o);
    if (tensor_core_ok(xt, weight, o, residual)) {
        GemmFusion f;
        memset(&f, 0, sizeof f);
        fusion_in(x, f);
        return linear_tc(xt, weight, bias, residual, o, -1, -1, -1, 0, x.deferred ? &f : nullptr);
    }
    Tensor xin = x.deferred ? materialize(x) : xt;
    return linear_simt(xin, weight, bias, residual, o);
}

Tensor Ops::materialize(const Rows& h) {
    return h.deferred ? rmsnorm(h.source, h.weight, h.eps) : h.t;
}

std::pair<Tensor, Rows> Ops::linear_norm(const Rows& x, const Tensor& weight, const Tensor& norm_weight, float eps,
                                         const Tensor* bias, const Tensor* residual) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const int64_t rows = xt.rows(), n = weight.rows();
    if (norm_weight.numel() == n) {
        Tensor probe = Tensor::make((void*)16, xt.dtype, {rows, n});      // shape and alignment of a fresh result
        // few rows: the weights lie on the tiles' M side (the planner's choice up to 128 rows) and every tile of 128
        // columns adds one partial sum per row; many rows: the rows lie on the M side and every column tile adds one
        bool few = false, many = false;
        int bn = 0, swap = -1;
        if (tensor_core_ok(xt, weight, probe, residual)) {
            bool swapped = false;
            plan(rows, n, xt.cols(), &swapped, &bn);
            few = swapped && few_rows_tile_ok(xt, weight, probe, residual, 128);
            many = !few && n % 16 == 0 && few_rows_tile_ok(xt, weight, probe, residual, rows, 16);
            if (many && swapped) {
                // few rows whose width is no multiple of 128: the fused norm wants whole tiles that way round, so the
                // product runs the other way round
                long long p[8] = {0};
                const auto& g = kernels::gemm_tc();
                if (g.plan((int)rows, (int)n, (int)xt.cols(), sms_, 0, -1, -1, p) != 0)
                    throw KernelError(std::string("gemm_tc_plan: ") + g.last_error());
                bn = (int)p[1];
                swap = 0;
            }
        }
        if (few || many) {
            Tensor out = alloc(xt.dtype, rows, n);
            check_residual(residual, out);
            Tensor scaled = alloc(xt.dtype, rows, n);
            const int64_t parts = few ? n / 128 : (n + bn - 1) / bn;
            Tensor ssq = alloc(DType::F32, parts, rows);
            GemmFusion f;
            memset(&f, 0, sizeof f);
            fusion_in(x, f);
            f.norm_w = norm_weight.data;
            f.norm_w_dtype = code(norm_weight.dtype);
            f.norm_out = scaled.data;
            f.out_ssq = (float*)ssq.data;
            linear_tc(xt, weight, bias, residual, out, swap, -1, -1, 0, &f);
            Rows r;
            r.t = scaled;
            r.deferred = true;
            r.ssq = ssq;
            r.eps = eps;
            r.source = out;
            r.weight = norm_weight;
            return {out, r};
        }
    }
    Tensor out = linear(x, weight, bias, residual);
    return {out, Rows(rmsnorm(out, norm_weight, eps))};
}

Tensor Ops::qkv_rope_write(const Rows& x, const Tensor& weight, const Tensor* bias, const int* row_seq,
                           const int* row_pos, const float* denominators, int rotary_dim, int n_heads, int n_kv_heads,
                           int head_dim, const CacheView* view) {
    const Tensor& xt = x.t;
    check_product(xt, weight);
    const int64_t n = weight.rows();
    const bool write = view && view->write && view->k_pool;
    if (128 % head_dim == 0 && head_dim % 8 == 0 && n == (int64_t)(n_heads + 2 * n_kv_heads) * head_dim &&
        (!denominators || rotary_dim % 16 == 0)) {
        Tensor probe = Tensor::make((void*)16, xt.dtype, {xt.rows(), n});
        if (few_rows_tile_ok(xt, weight, probe, nullptr, 64) && (!write || view->dtype == DType::BF16)) {
            Tensor out = alloc(xt.dtype, xt.rows(), n);
            GemmFusion f;
            memset(&f, 0, sizeof f);
            fusion_in(x, f);
            f.row_seq = row_seq;
            f.row_pos = row_pos;
            f.denom = denominators;
            f.rot = denominators ? rotary_dim : 0;
            f.nq = n_heads;
            f.nkv = n_kv_heads;
            f.hd = head_dim;
            if (write) {
                f.k_pool = view->k_pool;
                f.v_pool = view->v_pool;
                f.table = view->block_table;
                f.table_width = view->table_width;
                f.page = view->page_size;
            }
            return linear_tc(xt, weight, bias, nullptr, out, -1, -1, -1, 0, &f);
        }
    }
    Tensor qkv = linear(x, weight, bias);
    if (denominators || write) rope_kv_write(qkv, row_seq, row_pos, denominators, rotary_dim, n_heads, n_kv_heads, head_dim, view);
    return qkv;
}

Tensor Ops::linear_swiglu(const Rows& x, const Tensor& weight_pairs, int act) {
    const Tensor& xt = x.t;
    check_product(xt, weight_pairs);
    const int64_t inner = weight_pairs.rows() / 2;
    Tensor probe = Tensor::make((void*)16, xt.dtype, {xt.rows(), inner});
    if (xt.dtype == DType::BF16 && tensor_core_ok(xt, weight_pairs, probe, nullptr)) {
        Tensor out = alloc(xt.dtype, xt.rows(), inner);
        GemmFusion f;
        memset(&f, 0, sizeof f);
        fusion_in(x, f);
        return linear_tc(xt, weight_pairs, nullptr, nullptr, out, -1, -1, -1, act, x.deferred ? &f : nullptr);
    }
    return swiglu(linear(x, weight_pairs), act);
}

// ------------------------------------------------------------------ attention
int Ops::attention_splits(int64_t rows, int n_heads, int max_kv_len) const {
    // CUDA-core kernel: few rows facing long contexts are cut along the keys so that the device fills.
    const int64_t warps = rows * n_heads, want = (int64_t)sms_ * 16;
    if (warps >= want || max_kv_len <= 128) return 1;
    int64_t s = want / (warps > 0 ? warps : 1);
    const int64_t blocks = (max_kv_len + 63) / 64;
    if (s > blocks) s = blocks;
    if (s > 64) s = 64;
    return (int)(s < 1 ? 1 : s);
}

// FRIDAY_ATTN_WIDE=0: the CTAs that share a sequence's keys in a one-token step always form one thread-block cluster.
static bool wide_splits() {
    const char* e = getenv("FRIDAY_ATTN_WIDE");
    return e == nullptr || e[0] != '0';
}

int Ops::decode_splits(int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_kv_len) {
    // How many CTAs share one sequence's keys in a one-token step: the number with the shortest estimated time.
    // Up to 8 they form a thread-block cluster and merge through each other's shared memory; 9 to 64 leave partial
    // rows in memory and the last to finish merges them.  The estimate, in us, fitted to one-token steps of 1 to 32
    // sequences with 2,000 to 32,000 keys on a B200 (28 query heads on 4 kv heads of 128):
    //  - a CTA streams a block of 64 keys in 0.84 us while it has its SM to itself; the more SMs hold two CTAs, the
    //    slower each gets (1.13 us when 108 of 148 SMs hold two);
    //  - the device says how many clusters of a size it holds when empty; SMs that the kernel before frees one by
    //    one are packed less well, the worse the larger the cluster (32 clusters of 8 ran in two waves although 33
    //    fit, 32 of 7 were slower than 32 of 6 although 37 fit), so 2 % less per CTA of a cluster count as one wave,
    //    and every wave costs its CTAs' set-up and the merge again (2.5 us and 0.15 us per CTA of a cluster; through
    //    memory 5 us and 0.2 us per CTA).
    const int group = n_heads / n_kv_heads;
    const long long base = (long long)n_seqs * n_kv_heads * ((group + 15) / 16);
    if (base < 1) return 1;
    if (const char* e = getenv("FRIDAY_ATTN_SPLITS")) {              // for measurements: this many, whatever the shape
        const int v = atoi(e);
        if (v >= 1 && v <= 64) return v;
    }
    const int blocks = (max_kv_len + 63) / 64;
    int top = blocks / 2 < 1 ? 1 : blocks / 2;                      // every CTA keeps at least two blocks
    if (top > 8) top = 8;
    auto fit_of = [&](int size) {
        auto key = std::make_pair(head_dim, size);
        auto it = cluster_fit_.find(key);
        if (it == cluster_fit_.end()) it = cluster_fit_.emplace(key, kernels::attention_mma().clusters_at_once(head_dim, size)).first;
        return (long long)((1.0 - 0.02 * size) * it->second);
    };
    auto per_block = [&](double resident) {
        const double second = resident > sms_ ? resident - sms_ : 0.0;
        return 0.84 * (1.0 + 0.47 * second / sms_);
    };
    double best = 1e30;
    int pick = 1;
    for (int size = 1; size <= top; ++size) {
        const long long fit = fit_of(size);
        if (fit < 1) continue;
        const int per = (blocks + size - 1) / size;
        double t = 0.0;
        for (long long left = base; left > 0;) {
            const long long now = left < fit ? left : fit;
            t += per * per_block((double)now * size) + 2.5 + 0.15 * size;
            left -= now;
        }
        if (t < best) {
            best = t;
            pick = size;
        }
    }
    if (wide_splits()) {
        const long long at_once = fit_of(1);
        for (int wide = 9; wide <= 64 && wide <= blocks / 3 && base * wide <= at_once; ++wide) {
            const double t = (blocks + wide - 1) / wide * per_block((double)base * wide) + 5.0 + 0.2 * wide;
            if (t < best) {
                best = t;
                pick = wide;
            }
        }
    }
    return pick;
}

void Ops::attention(const Tensor& q, int64_t q_stride, Tensor& out, const CacheView& view, const StepContext& ctx,
                    int n_heads, int n_kv_heads, int head_dim, int window, float scale, float out_scale) {
    if (view.kind != CacheRequest::KV || !view.k_pool) throw KernelError("attention needs a view of keys and values");
    const int vd = view.v_head_dim > 0 ? view.v_head_dim : head_dim;
    const int keep = window > 0 ? view.keep_first : 0;
    if (vd != head_dim || keep > 0 || out_scale != 1.0f) {
        // prompts in bf16: tensor cores (mma.sync), 32-bit softmax; FRIDAY_ATTN_WINDOW=0 keeps them on the CUDA cores
        if (out.dtype == DType::BF16 && !ctx.decode && ctx.seq_start != nullptr && env_on("FRIDAY_ATTN_WINDOW") &&
            head_dim <= 128 && vd <= 128 && view.page_size == 64) {
            const auto& k = kernels::attention_window();
            Timed t(*this, Attention);
            call(launches_, k,
                 k.run(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.block_table, view.table_width, view.page_size,
                       ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.n_seqs, ctx.max_q_len, n_heads, n_kv_heads, head_dim, vd, window,
                       keep, scale, out_scale, stream_),
                 "attention_window");
            return;
        }
        // the general form: CUDA cores, fp32 arithmetic
        const int rows_ = (int)out.rows();
        int kv_reach = ctx.max_kv_len;
        if (window > 0 && window + keep < kv_reach) kv_reach = window + keep;
        const int splits = attention_splits(rows_, n_heads, kv_reach);
        float* scratch = splits > 1 ? scratch_floats((int64_t)rows_ * n_heads * splits * (vd + 2)) : nullptr;
        const auto& k = kernels::attention_simt();
        Timed t(*this, Attention);
        call(launches_, k,
             k.masked(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.block_table, view.table_width, view.page_size,
                      ctx.row_seq, ctx.row_pos, rows_, n_heads, n_kv_heads, head_dim, vd, window, keep, scale, out_scale, splits,
                      scratch, code(out.dtype), stream_),
             "attention_simt_masked");
        return;
    }
    const bool geometry = ctx.seq_start != nullptr;
    const bool hd_ok = head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128 && view.page_size == 64;
    const int rows = (int)out.rows();
    if (out.dtype == DType::BF16 && geometry && !ctx.decode && attn_tc_ && hd_ok && n_kv_heads > 0 &&
        n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 128 && q_stride % 8 == 0) {
        const auto& k = kernels::attention_tc();
        Timed t(*this, Attention);
        call(launches_, k,
             k.run(q.data, (int)q_stride, (int)q.rows(), out.data, view.k_pool, view.v_pool, view.pool_pages,
                   view.block_table, view.table_width, ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.row_seq, ctx.n_seqs,
                   ctx.max_q_len, n_heads, n_kv_heads, head_dim, window, scale, (int*)status_.get(), stream_),
             "attention_tc");
        return;
    }
    if (out.dtype == DType::BF16 && geometry && hd_ok) {
        const bool keys_mode = ctx.decode;
        const int splits = keys_mode ? decode_splits(ctx.n_seqs, n_heads, n_kv_heads, head_dim, ctx.max_kv_len) : 1;
        float* scratch = splits > 1 ? scratch_floats((int64_t)rows * n_heads * splits * (head_dim + 2)) : nullptr;
        const auto& k = kernels::attention_mma();
        Timed t(*this, Attention);
        call(launches_, k,
             k.run(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.pool_pages, view.block_table,
                   view.table_width, 64, ctx.seq_start, ctx.seq_qlen, ctx.seq_pos0, ctx.row_seq, ctx.n_seqs, rows,
                   ctx.max_q_len, n_heads, n_kv_heads, head_dim, window, scale, keys_mode ? 1 : 0, splits, scratch,
                   (int*)attn_counters_.get(), (int)(attn_counters_.bytes() / sizeof(int)), (int*)status_.get(), stream_),
             "attention_mma");
        return;
    }
    const int splits = attention_splits(rows, n_heads, ctx.max_kv_len);
    float* scratch = splits > 1 ? scratch_floats((int64_t)rows * n_heads * splits * (head_dim + 2)) : nullptr;
    const auto& k = kernels::attention_simt();
    Timed t(*this, Attention);
    call(launches_, k,
         k.run(q.data, (int)q_stride, out.data, view.k_pool, view.v_pool, view.block_table, view.table_width,
               view.page_size, ctx.row_seq, ctx.row_pos, rows, n_heads, n_kv_heads, head_dim, window, scale, splits,
               scratch, code(out.dtype), stream_),
         "attention_simt");
}

// ------------------------------------------------------------------ sampling
void Ops::sample(const Tensor& logits, const float* temperature, const int* streams, const int* steps,
                 unsigned long long seed, const int* row_live, int* out) {
    if (logits.dtype != DType::F32) throw KernelError("sample: logits are float32");
    const auto& k = kernels::sampling();
    Timed t(*this, Other);
    call(launches_, k,
         k.sample((const float*)logits.data, (int)logits.rows(), (int)logits.cols(), (int)logits.ld, temperature, streams,
                  steps, seed, row_live, out, stream_),
         "sampling_sample");
}

void Ops::check_status() {
    int word[4] = {0, 0, 0, 0};
    cuda_check(cudaMemcpyAsync(word, status_.get(), sizeof word, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    if (word[0] != 0) {
        cuda_check(cudaMemsetAsync(status_.get(), 0, sizeof word, stream_), "cudaMemsetAsync");
        throw KernelError(format("a tensor-core kernel on device %d gave up waiting (code %d: which of its bounded waits, "
                                 "see gemm_tc.cu and attention_tc.cu); its results are not valid", device_, word[0]));
    }
}

}  // namespace friday
