// Parts beyond softmax attention and the dense feed-forward: two mixers that carry a matrix-valued state per head
// from token to token, a mixer that runs others side by side, routed experts, and a per-layer token input.
//
//   mixer "gated_linear_attention"   S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t,  a_t = sigmoid(z_t)^(1/tau)
//   mixer "shift_decay_mix"          each projection reads its own blend of the row and the row before it;
//                                    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,  S_t = diag(w_t) S_(t-1) + k_t v_t^T,
//                                    w_t = exp(-exp(z_t))
//   mixer "parallel"                 sum of scale_i * mixer_i(h) over members that read the same input, each with a cache
//                                    entry part of its own
//   feed_forward "routed_experts"    top-k of a biased router, weights by softmax over the chosen logits, gated experts; or
//                                    sigmoid scores with a choice bias and groups of experts, and an expert for every row
//   token_input "gated_token_table"  x += norm(proj(gelu_tanh(gate x) * table[token]))
//
// The states, the decays and everything that enters the recurrences besides the projections are fp32 (csrc/recurrence.cu);
// router logits, the choice and the weights are fp32 (csrc/routed.cu).  Every part adds into the residual stream that it
// is given, in that stream's dtype (32-bit floats for a model that keeps its stream so).
#include <math.h>
#include <stdlib.h>

#include <string>

#include "friday/ops.h"
#include "friday/parts.h"

namespace friday {

namespace {

// columns [c0, c0 + n) of a 2-d tensor, as a view with the same row stride
Tensor columns(const Tensor& t, int64_t c0, int64_t n) {
    Tensor v = t;
    v.data = (char*)t.data + (size_t)c0 * dtype_size(t.dtype);
    v.shape[1] = n;
    return v;
}

// A size that the checkpoint's tensor shapes give when the specification does not: -1 stands for "as stored".
int64_t given_or_stored(const PartSpec& s, const char* key) {
    const int64_t v = s.params.get_int(key, -1);
    return v > 0 ? v : -1;
}

int positive(const PartSpec& s, const char* key, const char* part) {
    const int64_t v = s.params.get_int(key, 0);
    if (v <= 0) throw ConfigError(format("%s needs a positive '%s'", part, key));
    return (int)v;
}

}  // namespace

// ------------------------------------------------------------------ gated linear attention
// q = Wq h / sqrt(dk), k = Wk h (heads x dk), v = Wv h (heads x dv); a decay per key channel a = sigmoid(z)^(1/tau) with
// z = Wa2 (Wa1 h) + b; per head S = diag(a) S + k v^T, o = S^T q; o is RMS-normed per head with a weight [dv] shared by
// the heads, multiplied by silu(Wg h) and projected by Wo.  q, k, v, the gate and the first decay projection are one
// product over stacked matrices.
class GatedLinearAttention : public Mixer {
public:
    GatedLinearAttention(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "gated_linear_attention");
        dk_ = positive(s, "dim", "gated_linear_attention");
        dv_ = (int)s.params.get_int("vdim", dk_);
        rank_ = given_or_stored(s, "decay_rank");      // inner size of the decay's two projections
        tau_ = (float)s.params.get_double("tau", 1.0);
        eps_ = (float)s.params.get_double("eps", 1e-5);
        if (!(tau_ > 0.f) || dv_ <= 0) throw ConfigError("gated_linear_attention: 'tau' and 'vdim' must be positive");
        const int64_t w = e.width, hk = (int64_t)heads_ * dk_, hv = (int64_t)heads_ * dv_;
        declare_stacked("w_in", 2 * hk + 2 * hv, w);
        declare("q", {hk, w}).stack("w_in", 0);
        declare("k", {hk, w}).stack("w_in", hk);
        declare("v", {hv, w}).stack("w_in", 2 * hk);
        declare("g", {hv, w}).stack("w_in", 2 * hk + hv);
        declare("a1", {rank_, w});
        declare("a2", {hk, rank_});
        declare("a2.b", {hk});
        declare("norm", {(int64_t)dv_}, false, true);
        declare("o", {w, hv});
    }
    CacheRequest cache_request() const override { return CacheRequest::state({(int64_t)heads_ * dk_ * dv_}, DType::F32); }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (tensor("a1").rows() != tensor("a2").cols()) throw ConfigError(prefix + ": the decay's two projections do not fit each other");
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        const int64_t hk = (int64_t)heads_ * dk_, hv = (int64_t)heads_ * dv_;
        Tensor x = ops.materialize(h);
        Tensor in = ops.linear(Rows(x), tensor("w_in"));
        Tensor q = columns(in, 0, hk), k = columns(in, hk, hk), v = columns(in, 2 * hk, hv), g = columns(in, 2 * hk + hv, hv);
        Tensor z = ops.linear(Rows(ops.linear(Rows(x), tensor("a1"))), tensor("a2"), nullptr, nullptr, (int)DType::F32);
        Ops::ScanSpec sp;
        sp.heads = heads_;
        sp.dk = dk_;
        sp.dv = dv_;
        sp.mode = 0;
        sp.q_scale = 1.0f / sqrtf((float)dk_);
        sp.tau = tau_;
        sp.z_bias = &tensor("a2.b");
        Tensor o = ops.state_scan(q, k, v, z, sp, view, ctx);
        Tensor y = ops.head_norm_gate(o, g, tensor("norm"), false, heads_, dv_, eps_, out_scale, x.dtype, ctx);
        return PartOut(ops.linear_residual(Rows(y), tensor("o"), nullptr, residual));
    }

private:
    int heads_, dk_, dv_;
    int64_t rank_;
    float tau_, eps_;
};

// ------------------------------------------------------------------ token-shift mixing with a data-dependent decay
// With h' the row before (zeros before a sequence's first row), each of r, k, v, g, w reads h + (h' - h) * mu_s.
// r, k, v = W_s mix_s (heads x dim), gate = silu(Wg mix_g), decay w = exp(-exp(Ww2 tanh(Ww1 mix_w) + w0)) per head and
// key channel.  Per head o = (S + diag(u) k v^T)^T r, then S = diag(w) S + k v^T.  Each head's o is divided by its root
// mean square, multiplied by a weight [heads * dim] and the gate, and projected by Wo.  The state of a sequence is its
// last row (width numbers) followed by the heads' matrices.
class ShiftDecayMix : public Mixer {
public:
    ShiftDecayMix(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        heads_ = positive(s, "heads", "shift_decay_mix");
        dim_ = positive(s, "dim", "shift_decay_mix");
        rank_ = given_or_stored(s, "decay_rank");      // inner size of the decay's two projections
        eps_ = (float)s.params.get_double("eps", 1e-5);
        const int64_t w = e.width, hd = (int64_t)heads_ * dim_;
        for (const char* m : {"r", "k", "v", "g", "w"}) declare(std::string("mu.") + m, {w});
        for (const char* m : {"r", "k", "v", "g"}) declare(m, {hd, w});
        declare("w1", {rank_, w});
        declare("w2", {hd, rank_});
        declare("w0", {hd});
        declare("u", {(int64_t)heads_, (int64_t)dim_});
        declare("norm", {hd}, false, true);
        declare("o", {w, hd});
    }
    CacheRequest cache_request() const override {
        return CacheRequest::state({env.width + (int64_t)heads_ * dim_ * dim_}, DType::F32);
    }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (tensor("w1").rows() != tensor("w2").cols()) throw ConfigError(prefix + ": the decay's two projections do not fit each other");
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        Tensor x = ops.materialize(h);
        const int64_t rows = x.rows();
        Tensor mixes = ops.shift_mix(x, {tensor("mu.r"), tensor("mu.k"), tensor("mu.v"), tensor("mu.g"), tensor("mu.w")}, view, ctx);
        Tensor r = ops.linear(Rows(mixes.row_slice(0, rows)), tensor("r"));
        Tensor k = ops.linear(Rows(mixes.row_slice(rows, rows)), tensor("k"));
        Tensor v = ops.linear(Rows(mixes.row_slice(2 * rows, rows)), tensor("v"));
        Tensor g = ops.linear(Rows(mixes.row_slice(3 * rows, rows)), tensor("g"));
        Tensor lw = ops.linear(Rows(mixes.row_slice(4 * rows, rows)), tensor("w1"));
        ops.tanh_rows(lw);
        Tensor z = ops.linear(Rows(lw), tensor("w2"), nullptr, nullptr, (int)DType::F32);
        const Tensor& u = tensor("u");
        Tensor bonus = Tensor::make(u.data, u.dtype, {u.numel()});
        Ops::ScanSpec sp;
        sp.heads = heads_;
        sp.dk = dim_;
        sp.dv = dim_;
        sp.mode = 1;
        sp.state_offset = env.width;
        sp.z_bias = &tensor("w0");
        sp.bonus = &bonus;
        sp.carry = &x;
        Tensor o = ops.state_scan(r, k, v, z, sp, view, ctx);
        Tensor y = ops.head_norm_gate(o, g, tensor("norm"), true, heads_, dim_, eps_, out_scale, x.dtype, ctx);
        return PartOut(ops.linear_residual(Rows(y), tensor("o"), nullptr, residual));
    }

private:
    int heads_, dim_;
    int64_t rank_;
    float eps_;
};

// ------------------------------------------------------------------ mixers side by side
// out = residual + sum_i scale_i * member_i(h).  Members are named by the specification's "members" (roles of sub-parts,
// in order) and weighted by "scales"; each keeps the part of the cache entry that it asked for (a member that asks for
// several parts gets them as a view of several).  With "member_norms" (a tensor name [width] per member) every member's
// result is first RMS-normed over the width with that weight ("eps"): out = residual + sum_i scale_i * norm_i(member_i(h));
// the members then return their results alone, 32-bit, and the sum is one kernel for two members of equal scale.
class ParallelMixer : public Mixer {
public:
    ParallelMixer(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        const Json* members = s.params.find("members");
        const Json* scales = s.params.find("scales");
        if (!members || !members->is_array() || members->size() == 0 || !scales || !scales->is_array() ||
            scales->size() != members->size())
            throw ConfigError("parallel mixer needs 'members' (roles of its sub-parts) and as many 'scales'");
        for (size_t i = 0; i < members->size(); ++i) {
            const PartSpec& ms = s.part((*members)[i].as_string());
            members_.push_back(adopt(ms.prefix, build<Mixer>("mixer", ms, e)));
            scales_.push_back((float)(*scales)[i].as_double());
        }
        const Json* norms = s.params.find("member_norms");
        if (norms && norms->is_array()) {
            if (norms->size() != members->size()) throw ConfigError("parallel mixer: 'member_norms' names a tensor for every member");
            eps_ = (float)s.params.get_double("eps", 1e-5);
            for (size_t i = 0; i < norms->size(); ++i) {
                norm_names_.push_back((*norms)[i].as_string());
                declare(norm_names_.back(), {e.width}, false, true);
            }
        }
    }
    CacheRequest cache_request() const override {
        std::vector<CacheRequest> parts;
        for (const Mixer* m : members_) parts.push_back(m->cache_request());
        return CacheRequest::flat(parts);
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, Norm*) override {
        std::vector<CacheView> views;
        size_t at = 0;
        for (const Mixer* m : members_) {
            const CacheRequest r = m->cache_request();
            if (r.kind == CacheRequest::None) {
                views.emplace_back();
                at += 1;
                continue;
            }
            views.push_back(view.member(at, r));
            at += CacheRequest::flat_size(r);
        }
        if (view.kind != CacheRequest::Several || view.parts.size() != at)
            throw KernelError("parallel mixer: the cache view does not have a part per member");
        Rows x(ops.materialize(h));
        if (!norm_names_.empty()) {
            if (!residual.defined() || residual.dtype != DType::F32) throw ConfigError("parallel mixer: normed members add into a 32-bit residual stream");
            std::vector<Tensor> ys;
            for (size_t i = 0; i < members_.size(); ++i) {
                members_[i]->out_scale = 1.0f;
                ys.push_back(members_[i]->forward(ops, x, Tensor(), ctx, views[i], nullptr).x);
                if (ys.back().dtype != DType::F32) throw ConfigError("parallel mixer: a member handed no residual must return 32-bit rows");
            }
            if (members_.size() == 2 && scales_[0] == scales_[1])
                return PartOut(ops.rms_pair_add(residual, ys[0], ys[1], tensor(norm_names_[0]), tensor(norm_names_[1]), eps_, out_scale * scales_[0]));
            Tensor sum = residual;
            for (size_t i = 0; i < members_.size(); ++i) sum = ops.post_norm_add(sum, ys[i], tensor(norm_names_[i]), eps_, out_scale * scales_[i]);
            return PartOut(sum);
        }
        Tensor sum = residual;
        for (size_t i = 0; i < members_.size(); ++i) {
            members_[i]->out_scale = out_scale * scales_[i];
            sum = members_[i]->forward(ops, x, sum, ctx, views[i], nullptr).x;
        }
        return PartOut(sum);
    }

private:
    std::vector<Mixer*> members_;
    std::vector<float> scales_;
    std::vector<std::string> norm_names_;
    float eps_ = 1e-5f;
};

// ------------------------------------------------------------------ routed experts
// Router logits z = Wr h + b in fp32; the `top` largest are chosen, their weights are the softmax over the chosen logits
// (or over all of them with "softmax_all").  Expert e: Wd_e (silu(Wg_e h) * (Wu_e h)).  The experts' gate and up matrices
// are kept stacked row by row in turn, expert after expert, and their down matrices side by side, so that
//   few rows:   only the chosen experts' weights are read, once per (row, choice);
//   many rows:  either the rows are gathered expert by expert and every expert runs its two products over its own rows
//               (prompts; the host reads the row counts), or ALL experts run as one gated product on the tensor cores,
//               the result is multiplied by the routing weight (zero for an expert that was not chosen) and one product
//               over the down matrices side by side sums the chosen experts: experts / top times the arithmetic in two
//               launches.  Whichever is estimated to be less work runs.
class RoutedExperts : public FeedForward {
public:
    RoutedExperts(const PartSpec& s, const BuildEnv& e) : FeedForward(e) {
        experts_ = positive(s, "experts", "routed_experts");
        top_ = positive(s, "top", "routed_experts");
        inner_ = positive(s, "inner", "routed_experts");
        softmax_all_ = s.params.get_bool("softmax_all", false);
        if (top_ > experts_) throw ConfigError(format("routed_experts: top %d of %d experts", top_, experts_));
        if (top_ > 32 || experts_ > 256) throw ConfigError("routed_experts: at most 256 experts and 32 choices");
        // "score": "sigmoid" makes the scores sigmoid(logit): the choice runs on score + the tensor "choice_bias" (if named)
        // among the experts of the "groups_keep" best of "groups" equally sized runs of adjacent experts (a group counts as the sum of its
        // two largest), the weights are score * "weight_scale", not renormalised.  "router_bias": false leaves the logits'
        // bias out.  "shared_inner" > 0 adds an expert of that inner size ("shared.") that every row uses.
        const std::string score = s.params.get_string("score", "softmax");
        if (score != "softmax" && score != "sigmoid") throw ConfigError("routed_experts: 'score' is \"softmax\" or \"sigmoid\"");
        sigmoid_ = score == "sigmoid";
        router_bias_ = s.params.get_bool("router_bias", true);
        choice_bias_ = s.params.get_string("choice_bias", "");
        groups_ = (int)s.params.get_int("groups", 1);
        keep_ = (int)s.params.get_int("groups_keep", groups_);
        weight_scale_ = (float)s.params.get_double("weight_scale", 1.0);
        shared_inner_ = s.params.get_int("shared_inner", 0);
        if (groups_ < 1 || experts_ % groups_ || keep_ < 1 || keep_ > groups_ || keep_ * (experts_ / groups_) < top_)
            throw ConfigError(format("routed_experts: %d experts in %d groups of which %d are kept cannot give %d choices", experts_,
                                     groups_, keep_, top_));
        if (!sigmoid_ && (groups_ > 1 || !choice_bias_.empty() || weight_scale_ != 1.0f))
            throw ConfigError("routed_experts: groups, a choice bias and a weight multiplier belong to sigmoid scores");
        const int64_t w = e.width;
        declare("router", {(int64_t)experts_, w});
        if (router_bias_) declare("router.b", {(int64_t)experts_});
        if (!choice_bias_.empty()) declare(choice_bias_, {(int64_t)experts_});
        if (shared_inner_ > 0) {
            declare_stacked("w_shared", 2 * shared_inner_, w);
            declare("shared.gate", {shared_inner_, w}).stack("w_shared", 0, 2);
            declare("shared.up", {shared_inner_, w}).stack("w_shared", 1, 2);
            declare("shared.down", {w, shared_inner_});
        }
        declare_stacked("w_gate_up", (int64_t)experts_ * 2 * inner_, w);
        declare_stacked("w_down", w, (int64_t)experts_ * inner_);
        for (int x = 0; x < experts_; ++x) {
            const std::string p = format("e%d.", x);
            declare(p + "gate", {(int64_t)inner_, w}).stack("w_gate_up", (int64_t)x * 2 * inner_, 2);
            declare(p + "up", {(int64_t)inner_, w}).stack("w_gate_up", (int64_t)x * 2 * inner_ + 1, 2);
            declare(p + "down", {w, (int64_t)inner_}).stack_columns("w_down", (int64_t)x * inner_);
        }
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual_in, const StepContext& ctx, Norm*) override {
        Tensor x = ops.materialize(h);
        Tensor logits = ops.linear(Rows(x), tensor("router"), router_bias_ ? &tensor("router.b") : nullptr, nullptr, (int)DType::F32);
        // what the chosen experts' results are added to: the stream; with an expert that every row uses, its result on top
        // of the stream; without a stream (a block that sums itself), that result alone or zeros, 32-bit
        Tensor residual = residual_in;
        if (shared_inner_ > 0) {
            Tensor act = ops.linear_swiglu(Rows(x), tensor("w_shared"));
            if (residual.defined()) residual = ops.linear_residual(Rows(act), tensor("shared.down"), nullptr, residual);
            else residual = ops.linear(Rows(act), tensor("shared.down"), nullptr, nullptr, (int)DType::F32);
        } else if (!residual.defined()) {
            residual = ops.alloc(DType::F32, x.rows(), x.cols());
            cuda_check(cudaMemsetAsync(residual.data, 0, residual.bytes(), ops.stream()), "cudaMemsetAsync");
        }
        const bool tensor_cores = x.dtype == DType::BF16 && x.rows() > 32 && tensor("w_gate_up").dtype == DType::BF16 &&
                                  x.cols() % 8 == 0 && inner_ % 8 == 0;
        // Arithmetic of the dense form against the grouped one, in units of a product's multiply-adds: all experts for
        // every row, or the chosen ones plus what two launches per expert and the host's wait cost (measured on a B200:
        // grouping broke even at width 2,048 with 8 experts of inner size 2,048, 2 chosen, 2,048 rows, and won a fifth
        // of the prompt's time at width 4,096; a launch counts as 25 G multiply-adds, the wait as 100 G).  Grouping
        // needs the host, so a one-token step (which may be captured in a graph) never groups.
        const double per_row = 3.0 * (double)inner_ * (double)x.cols();
        const double dense_work = (double)x.rows() * experts_ * per_row;
        const double grouped_work = (double)x.rows() * top_ * per_row + (2.0 * experts_ * 25e9 + 100e9) / 2.0;
        // FRIDAY_EXPERTS=grouped|dense|pairs forces a form where it can run (for comparisons and tests)
        const char* force = getenv("FRIDAY_EXPERTS");
        const std::string forced = force ? force : "";
        const bool may_group = tensor_cores && !ctx.decode && ctx.rows == (int)x.rows() && ctx.n_seqs > 0;
        const bool grouped = may_group && (forced == "grouped" || (forced.empty() && grouped_work < dense_work));
        const bool dense = tensor_cores && !grouped && (forced == "dense" || (forced.empty() && experts_ <= 16 * top_));
        Ops::Routing r = sigmoid_ ? ops.route_scored(logits, top_, choice_bias_.empty() ? nullptr : &tensor(choice_bias_), groups_, keep_,
                                                     weight_scale_, dense)
                                  : ops.route(logits, top_, softmax_all_, dense);
        if (grouped) return PartOut(ops.experts_grouped(x, r, tensor("w_gate_up"), tensor("w_down"), residual, top_, inner_));
        if (dense) {
            Tensor act = ops.linear_swiglu(Rows(x), tensor("w_gate_up"));
            ops.scale_by_route(act, r.dense, experts_, inner_);
            return PartOut(ops.linear_residual(Rows(act), tensor("w_down"), nullptr, residual));
        }
        Tensor act = ops.expert_gate_up(x, r, tensor("w_gate_up"), top_, inner_);
        return PartOut(ops.expert_down_combine(act, r, tensor("w_down"), residual, top_, inner_));
    }

private:
    int experts_, top_, inner_;
    bool softmax_all_;
    bool sigmoid_ = false, router_bias_ = true;
    std::string choice_bias_;
    int groups_ = 1, keep_ = 1;
    float weight_scale_ = 1.0f;
    int64_t shared_inner_ = 0;
};

// ------------------------------------------------------------------ per-layer token input
// e = table[token][slice .. slice + dim), g = gelu_tanh(Wgate x) * e, y = Wproj g, x += y / rms(y) * norm.  The table is
// the model's (a shared tensor: every layer reads its own columns); the stream is 32-bit.
class GatedTokenTable : public TokenInput {
public:
    GatedTokenTable(const PartSpec& s, const BuildEnv& e) : TokenInput(e) {
        dim_ = positive(s, "dim", "gated_token_table");
        slice_ = s.params.get_int("slice", 0);
        eps_ = (float)s.params.get_double("eps", 1e-5);
        table_name_ = s.params.get_string("table", "");
        if (table_name_.empty() || slice_ < 0) throw ConfigError("gated_token_table needs 'table' (a shared tensor) and a slice");
        declare("gate", {(int64_t)dim_, e.width});
        declare("proj", {e.width, (int64_t)dim_});
        declare("norm", {e.width}, false, true);
    }
    void bind_shared(const std::map<std::string, Tensor>& shared) override {
        TokenInput::bind_shared(shared);
        auto it = shared.find(table_name_);
        if (it == shared.end()) throw ConfigError("gated_token_table: the model has no shared tensor '" + table_name_ + "'");
        table_ = it->second;
    }
    void forward(Ops& ops, Tensor& x, const StepContext& ctx) override {
        if (!table_.defined()) throw KernelError("gated_token_table: the token table was never bound");
        ops.token_input(x, ctx, table_, slice_ * dim_, tensor("gate"), tensor("proj"), tensor("norm"), eps_);
    }

private:
    int dim_;
    int64_t slice_;
    float eps_;
    std::string table_name_;
    Tensor table_;
};

namespace {
PartRegistrar s1("mixer", "gated_linear_attention", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GatedLinearAttention(s, e); });
PartRegistrar s2("mixer", "shift_decay_mix", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new ShiftDecayMix(s, e); });
PartRegistrar s3("mixer", "parallel", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new ParallelMixer(s, e); });
PartRegistrar s4("feed_forward", "routed_experts", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RoutedExperts(s, e); });
PartRegistrar s5("token_input", "gated_token_table", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GatedTokenTable(s, e); });
}  // namespace

}  // namespace friday
