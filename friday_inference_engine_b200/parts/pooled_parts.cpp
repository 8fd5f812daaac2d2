// Two more mixers: softmax attention behind a window with pooled blocks, a sink and a query multiplier, and the
// generalized delta rule.
//
//   mixer "pooled_attention"   q = Wq h (heads x dim), k = Wk h (kv_heads x dim), v = Wv h (kv_heads x vdim), or, with
//                              "values": "keys", v = k as projected and no Wv; "qk_norm": q and k heads are RMS-normed with
//                              the weights "q.norm" / "k.norm" [dim] shared by the heads; the position part may rotate the
//                              pairs (i, i + dims / 2) of q and k; row i sees token j if 0 <= i - j < "window" (0: every
//                              j <= i) and, with "pool" = P > 0, one mean key and mean value for each block of P tokens that
//                              lies wholly before the window (b P + P - 1 <= i - window), the means taken over the keys and
//                              values as the cache keeps them; scores (q . k) * "scale", times 1 + coef * ln(floor((i + 1) /
//                              every) + 1) with "q_temp": {coef, every}; "sink": exp(sink_h) joins head h's denominator
//                              (tensor "sink" [heads]); then Wo.  The cache keeps the window's keys and values per token and,
//                              with pooled blocks, a 32-bit row of sums per block.
//   mixer "general_delta"      r, k, v = W h (heads x dim); decay w = exp(-rate * sigmoid(Ww2 tanh(Ww1 h) + w0)) and removal
//                              a = sigmoid(Wa h + a.b) per head and key channel; with the unit key u = k / sqrt(sum k^2 + 1e-6):
//                              S <- diag(w) S - (a u)(u^T S) + k v^T (both terms read the old S), o = S^T r; every head's o
//                              is divided by its root mean square, multiplied by "norm" [heads * dim] and sigmoid(Wg h), then
//                              Wo.  State per sequence: the heads' matrices, fp32.
//
// Scores, softmax weights, norms, angles, decays, removal rates, unit keys and states are fp32 (csrc/attention_pooled.cu,
// csrc/delta.cu).  Handed an undefined residual, a mixer returns its result alone as 32-bit rows.
#include <math.h>

#include <string>

#include "friday/ops.h"
#include "friday/parts.h"

namespace friday {

namespace {

Tensor columns(const Tensor& t, int64_t c0, int64_t n) {
    Tensor v = t;
    v.data = (char*)t.data + (size_t)c0 * dtype_size(t.dtype);
    v.shape[1] = n;
    return v;
}

int positive(const PartSpec& s, const char* key, const char* part) {
    const int64_t v = s.params.get_int(key, 0);
    if (v <= 0) throw ConfigError(format("%s needs a positive '%s'", part, key));
    return (int)v;
}

// residual + scale * (y Wo^T), or the product alone in 32-bit where the caller sums
PartOut project_out(Ops& ops, const Tensor& y, const Tensor& w_o, const Tensor& residual, float scale) {
    if (!residual.defined()) {
        Tensor out = ops.linear(Rows(y), w_o, nullptr, nullptr, (int)DType::F32);
        if (scale != 1.0f) ops.scale_rows(out, scale);
        return PartOut(out);
    }
    return PartOut(ops.linear_residual(Rows(y), w_o, nullptr, residual, scale));
}

}  // namespace

// ------------------------------------------------------------------ attention with pooled blocks
class PooledAttention : public Mixer {
public:
    PooledAttention(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "pooled_attention");
        kv_heads_ = (int)s.params.get_int("kv_heads", heads_);
        dim_ = positive(s, "dim", "pooled_attention");
        vdim_ = (int)s.params.get_int("vdim", dim_);
        window_ = (int)s.params.get_int("window", 0);
        pool_ = (int)s.params.get_int("pool", 0);
        scale_ = (float)s.params.get_double("scale", 1.0 / sqrt((double)dim_));
        eps_ = (float)s.params.get_double("eps", 1e-5);
        has_sink_ = s.params.get_bool("sink", false);
        qk_norm_ = s.params.get_bool("qk_norm", false);
        const std::string values = s.params.get_string("values", "own");
        if (values != "own" && values != "keys") throw ConfigError("pooled_attention: 'values' is \"own\" or \"keys\"");
        shared_ = values == "keys";
        if (kv_heads_ <= 0 || heads_ % kv_heads_) throw ConfigError(format("pooled_attention: %d heads cannot share %d key/value heads", heads_, kv_heads_));
        if (dim_ > 256 || vdim_ <= 0 || vdim_ > 256) throw ConfigError("pooled_attention: head sizes of 1 to 256");
        if (shared_ && vdim_ != dim_) throw ConfigError(format("pooled_attention: values that are the keys have the keys' size (dim %d, vdim %d)", dim_, vdim_));
        if (window_ < 0 || pool_ < 0) throw ConfigError("pooled_attention: 'window' and 'pool' must not be negative");
        if (pool_ > 0 && window_ == 0) throw ConfigError("pooled_attention: pooled blocks lie before a window; without a window every token is seen");
        const Json* qt = s.params.find("q_temp");
        if (qt && qt->is_object()) {
            temp_coef_ = (float)qt->get_double("coef", 0.0);
            temp_every_ = (int)qt->get_int("every", 0);
            if (temp_every_ <= 0) throw ConfigError("pooled_attention: 'q_temp' needs a positive 'every'");
        }
        position_ = adopt("", build<Position>("position", s.part("position"), e));
        const int64_t w = e.width, qd = (int64_t)heads_ * dim_, kd = (int64_t)kv_heads_ * dim_, vd = shared_ ? 0 : (int64_t)kv_heads_ * vdim_;
        declare_stacked("w_in", qd + kd + vd, w);
        declare("q", {qd, w}).stack("w_in", 0);
        declare("k", {kd, w}).stack("w_in", qd);
        if (!shared_) declare("v", {vd, w}).stack("w_in", qd + kd);
        if (qk_norm_) {
            declare("q.norm", {(int64_t)dim_}, false, true);
            declare("k.norm", {(int64_t)dim_}, false, true);
        }
        if (has_sink_) declare("sink", {(int64_t)heads_});
        declare("o", {w, (int64_t)heads_ * vdim_});
    }
    CacheRequest cache_request() const override {
        CacheRequest tokens = CacheRequest::kv(kv_heads_, dim_, window_, vdim_, 0);
        tokens.keys_only = shared_;
        if (pool_ == 0) return tokens;
        CacheRequest blocks = CacheRequest::kv(kv_heads_, dim_, 0, vdim_, 0);
        blocks.every = pool_;
        blocks.store_f32 = true;
        blocks.keys_only = false;
        return CacheRequest::several({tokens, blocks});
    }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        const float* denominators = nullptr;
        int d = 0;
        if (position_->halves(&freq_, &rot_mult_, &rot_)) {
            if (rot_ > dim_ || rot_ % 2) throw ConfigError(format("%s: %d rotated numbers in heads of %d", prefix.c_str(), rot_, dim_));
        } else if (position_->rotary(&denominators, &d) || position_->pairs(&freq_, &rot_mult_, &d)) {
            throw ConfigError(prefix + ": pooled_attention takes a position part that turns the pairs (i, i + dims / 2), or none");
        }
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        const CacheView* tokens = &view;
        const CacheView* blocks = nullptr;
        if (pool_ > 0) {
            if (view.kind != CacheRequest::Several || view.parts.size() != 2) throw KernelError("pooled_attention: the cache view lacks the tokens' part or the blocks'");
            tokens = &view.parts[0];
            blocks = &view.parts[1];
        }
        Tensor in = ops.linear(h, tensor("w_in"));
        Ops::PooledSpec sp;
        sp.heads = heads_;
        sp.kv_heads = kv_heads_;
        sp.dim = dim_;
        sp.vdim = vdim_;
        sp.window = window_;
        sp.pool = pool_;
        sp.scale = scale_;
        sp.temp_coef = temp_coef_;
        sp.temp_every = temp_every_;
        sp.sink = has_sink_ ? &tensor("sink") : nullptr;
        sp.q_norm = qk_norm_ ? &tensor("q.norm") : nullptr;
        sp.k_norm = qk_norm_ ? &tensor("k.norm") : nullptr;
        sp.eps = eps_;
        sp.freq = freq_;
        sp.rot_mult = rot_mult_;
        sp.rot = rot_;
        sp.q_off = 0;
        sp.k_off = (int64_t)heads_ * dim_;
        sp.v_off = shared_ ? -1 : sp.k_off + (int64_t)kv_heads_ * dim_;
        ops.pooled_store(in, sp, *tokens, blocks, ctx);
        Tensor mixed = ops.pooled_attention(in, sp, *tokens, blocks, ctx);
        return project_out(ops, mixed, tensor("o"), residual, out_scale);
    }

private:
    int heads_, kv_heads_, dim_, vdim_, window_, pool_, temp_every_ = 0, rot_ = 0;
    float scale_, eps_, temp_coef_ = 0.f, rot_mult_ = 1.0f;
    bool has_sink_, qk_norm_, shared_;
    Position* position_;
    const float* freq_ = nullptr;
};

// ------------------------------------------------------------------ generalized delta rule
class GeneralDelta : public Mixer {
public:
    GeneralDelta(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "general_delta");
        dim_ = positive(s, "dim", "general_delta");
        eps_ = (float)s.params.get_double("eps", 1e-5);
        rate_ = (float)s.params.get_double("rate", exp(-0.5));
        if (dim_ > 256) throw ConfigError("general_delta: at most 256 channels per head");
        const int64_t rank = s.params.get_int("decay_rank", -1) > 0 ? s.params.get_int("decay_rank", -1) : -1;     // else the checkpoint's
        const int64_t w = e.width, hd = (int64_t)heads_ * dim_;
        declare_stacked("w_in", 4 * hd, w);                      // one product for r, k, v and the gate
        declare("r", {hd, w}).stack("w_in", 0);
        declare("k", {hd, w}).stack("w_in", hd);
        declare("v", {hd, w}).stack("w_in", 2 * hd);
        declare("g", {hd, w}).stack("w_in", 3 * hd);
        declare("a", {hd, w});
        declare("a.b", {hd});
        declare("w1", {rank, w});
        declare("w2", {hd, rank});
        declare("w0", {hd});
        declare("norm", {hd}, false, true);
        declare("o", {w, hd});
    }
    CacheRequest cache_request() const override { return CacheRequest::state({(int64_t)heads_ * dim_ * dim_}, DType::F32); }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (tensor("w1").rows() != tensor("w2").cols()) throw ConfigError(prefix + ": the decay's two projections do not fit each other");
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        const int64_t hd = (int64_t)heads_ * dim_;
        Tensor x = ops.materialize(h);
        Tensor in = ops.linear(Rows(x), tensor("w_in"));
        // what enters the recurrence stays 32-bit: the removal's and the decay's raw projections
        Tensor a_raw = ops.linear(Rows(x), tensor("a"), nullptr, nullptr, (int)DType::F32);
        Tensor lw = ops.linear(Rows(x), tensor("w1"));
        ops.tanh_rows(lw);
        Tensor z = ops.linear(Rows(lw), tensor("w2"), nullptr, nullptr, (int)DType::F32);
        Ops::GeneralDeltaSpec sp;
        sp.heads = heads_;
        sp.dk = dim_;
        sp.dv = dim_;
        sp.rate = rate_;
        sp.unit_eps = 1e-6f;
        sp.r_off = 0;
        sp.k_off = hd;
        sp.v_off = 2 * hd;
        Tensor o = ops.general_delta(in, z, a_raw, tensor("w0"), tensor("a.b"), sp, view, ctx);
        Tensor y = ops.head_norm_gate(o, columns(in, 3 * hd, hd), tensor("norm"), true, heads_, dim_, eps_, 1.0f, x.dtype, ctx, true);
        return project_out(ops, y, tensor("o"), residual, out_scale);
    }

private:
    int heads_, dim_;
    float eps_, rate_;
};

namespace {
PartRegistrar p1("mixer", "pooled_attention", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new PooledAttention(s, e); });
PartRegistrar p2("mixer", "general_delta", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GeneralDelta(s, e); });
}  // namespace

}  // namespace friday
