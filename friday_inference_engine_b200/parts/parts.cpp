// The registry of parts, the description of a model as data, and the parts this library
// ships: RMSNorm, layer norm, rotary encodings (NeoX halves, neighbouring pairs with stretched wavelengths, and "none"),
// grouped-query attention, the SwiGLU
// feed-forward and the pre-norm residual block.
#include "friday/parts.h"

#include <dlfcn.h>
#include <math.h>

#include <algorithm>
#include <mutex>

#include "friday/ops.h"

namespace friday {

// ------------------------------------------------------------------ specs
const PartSpec& PartSpec::part(const std::string& role) const {
    auto it = parts.find(role);
    if (it == parts.end()) throw ConfigError("part '" + kind + "' needs a sub-part '" + role + "' in its specification");
    return it->second;
}

std::map<int, int> ModelSpec::cache_entries() const {
    std::map<int, int> owners;
    for (size_t i = 0; i < program.size(); ++i) {
        const LayerCall& c = program[i];
        if (c.layer < 0 || c.layer >= (int)layers.size())
            throw ConfigError(format("program entry %zu names layer %d of %zu", i, c.layer, layers.size()));
        if (c.cache < 0 || !c.write) continue;
        if (owners.count(c.cache))
            throw ConfigError(format("cache entry %d is written by program entries %d and %zu", c.cache, owners[c.cache], i));
        owners[c.cache] = (int)i;
    }
    for (size_t i = 0; i < program.size(); ++i) {
        const LayerCall& c = program[i];
        if (c.cache >= 0 && !c.write && (!owners.count(c.cache) || owners[c.cache] > (int)i))
            throw ConfigError(format("program entry %zu reads cache entry %d before anything wrote it", i, c.cache));
    }
    return owners;
}

CacheRequest CacheRequest::kv(int n_kv_heads, int head_dim, int window, int v_head_dim, int keep_first) {
    CacheRequest r;
    r.kind = KV;
    r.n_kv_heads = n_kv_heads;
    r.head_dim = head_dim;
    r.window = window;
    r.v_head_dim = v_head_dim == head_dim ? 0 : v_head_dim;
    r.keep_first = window > 0 ? keep_first : 0;
    return r;
}

CacheRequest CacheRequest::several(const std::vector<CacheRequest>& parts) {
    CacheRequest r;
    r.kind = Several;
    r.parts = parts;
    return r;
}

CacheRequest CacheRequest::flat(const std::vector<CacheRequest>& members) {
    CacheRequest r;
    r.kind = Several;
    for (const CacheRequest& m : members) {
        if (m.kind != Several) {
            r.parts.push_back(m);
            continue;
        }
        for (const CacheRequest& p : m.parts) {
            if (p.kind == Several) throw ConfigError("a cache request nests requests of several parts more than one level deep");
            r.parts.push_back(p);
        }
    }
    return r;
}

CacheView CacheView::member(size_t first, const CacheRequest& request) const {
    const size_t count = CacheRequest::flat_size(request);
    if (kind != CacheRequest::Several || first + count > parts.size()) throw KernelError("a cache view does not have the parts that its request was made of");
    if (request.kind != CacheRequest::Several) return parts[first];
    CacheView v;
    v.kind = CacheRequest::Several;
    v.write = write;
    v.parts.assign(parts.begin() + (long)first, parts.begin() + (long)(first + count));
    return v;
}

CacheRequest CacheRequest::state(const std::vector<int64_t>& shape, DType dtype) {
    CacheRequest r;
    r.kind = State;
    r.state_shape = shape;
    r.state_dtype = dtype;
    return r;
}

// ------------------------------------------------------------------ Part
ParamDecl& Part::declare(const std::string& name, const std::vector<int64_t>& shape, bool integer, bool one) {
    ParamDecl d;
    d.shape = shape;
    d.integer = integer;
    d.one = one;
    params.emplace_back(name, d);
    return params.back().second;
}

const Tensor& Part::tensor(const std::string& name) const {
    auto it = tensors.find(name);
    if (it == tensors.end() || !it->second.defined())
        throw KernelError("part parameter '" + prefix + name + "' was never set (the model's weights are not loaded)");
    return it->second;
}

void Part::finalize(Ops& ops) {
    for (auto& c : children_) c.second->finalize(ops);
}

void Part::bind_shared(const std::map<std::string, Tensor>& shared) {
    for (auto& c : children_) c.second->bind_shared(shared);
}

void Part::named_params(const std::string& pre, std::vector<Named>& out) {
    for (auto& p : params) out.push_back(Named{pre + p.first, this, p.first, p.second});
    for (auto& c : children_) c.second->named_params(pre + c.first, out);
}

// ------------------------------------------------------------------ registry
namespace {
const char* kCategories[] = {"norm", "position", "mixer", "feed_forward", "token_input", "block"};
std::mutex& reg_mutex() { static std::mutex m; return m; }
std::map<std::string, std::map<std::string, PartFactory>>& reg() {
    static std::map<std::string, std::map<std::string, PartFactory>> r;
    return r;
}
bool known_category(const std::string& c) {
    for (const char* k : kCategories)
        if (c == k) return true;
    return false;
}
}  // namespace

void register_part(const std::string& category, const std::string& kind, PartFactory factory) {
    if (!known_category(category))
        throw ConfigError("unknown part category '" + category + "' (have: norm, position, mixer, feed_forward, token_input, block)");
    std::lock_guard<std::mutex> lock(reg_mutex());
    reg()[category][kind] = std::move(factory);
}

std::vector<std::string> registered_parts(const std::string& category) {
    if (!known_category(category))
        throw ConfigError("unknown part category '" + category + "' (have: norm, position, mixer, feed_forward, token_input, block)");
    std::lock_guard<std::mutex> lock(reg_mutex());
    std::vector<std::string> out;
    for (const auto& kv : reg()[category]) out.push_back(kv.first);
    return out;
}

Part* build_part(const std::string& category, const PartSpec& spec, const BuildEnv& env) {
    PartFactory f;
    {
        std::lock_guard<std::mutex> lock(reg_mutex());
        auto& kinds = reg()[category];
        auto it = kinds.find(spec.kind);
        if (it == kinds.end()) {
            std::string known;
            for (const auto& kv : kinds) known += (known.empty() ? "" : ", ") + kv.first;
            throw ConfigError("no " + category + " part named '" + spec.kind + "' (registered: " +
                              (known.empty() ? "none" : known) + ")");
        }
        f = it->second;
    }
    Part* p = f(spec, env);
    p->prefix = spec.prefix;
    return p;
}

void load_plugin(const std::string& path) {
    if (!dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL))
        throw Error(ErrorKind::Other, "cannot load plug-in " + path + ": " + dlerror());
}

// ------------------------------------------------------------------ RMSNorm
// y = x / sqrt(mean(x^2) + eps) * weight, the mean taken in fp32.  Reference: rmsNormKernel
// (cuda_math_kernels.cu:280-321), friday_cpu::rmsNorm (cpu_ops.cpp:10-24).
class RMSNorm : public Norm {
public:
    RMSNorm(const PartSpec& s, const BuildEnv& e) : Norm(e) {
        const Json* eps = s.params.find("eps");
        if (!eps || !eps->is_number()) throw ConfigError("rmsnorm needs 'eps'");
        eps_ = (float)eps->as_double();
        width_ = s.params.get_int("width", e.width);
        // offset: the stored weight is a deviation from it (1 for weights kept around zero); the multiplier is
        // offset + weight, formed in fp32
        offset_ = (float)s.params.get_double("offset", 0.0);
        // out: "float32" writes 32-bit rows whatever the activations' dtype (a norm that feeds a 32-bit residual stream)
        const std::string out = s.params.get_string("out", "");
        if (!out.empty() && out != "float32") throw ConfigError("rmsnorm: 'out' is \"float32\" or absent");
        out_ = out.empty() ? e.dtype : DType::F32;
        declare(s.params.get_string("weight_name", "weight"), {width_}, false, offset_ == 0.f);
        name_ = s.params.get_string("weight_name", "weight");
    }
    Tensor forward(Ops& ops, const Tensor& x) override {
        if (offset_ == 0.f && x.dtype == out_) return ops.rmsnorm(x, tensor(name_), eps_);
        return ops.rmsnorm_to(x, tensor(name_), offset_, eps_, out_);
    }
    bool as_rmsnorm(Tensor* weight, float* eps) const override {
        if (offset_ != 0.f || out_ != env.dtype) return false;      // the products' fused norm knows plain weights only
        *weight = tensor(name_);
        *eps = eps_;
        return true;
    }
    bool rms_parts(Tensor* weight, float* eps) const override {
        if (offset_ != 0.f) return false;
        *weight = tensor(name_);
        *eps = eps_;
        return true;
    }

private:
    float eps_, offset_;
    int64_t width_;
    DType out_;
    std::string name_;
};

// ------------------------------------------------------------------ layer norm
// y = (x - mean) / sqrt(variance + eps) * weight + bias, mean and variance (the mean of the squared deviations) in fp32.
// The weight's tensor is "weight_name" (default "weight"), the bias "bias_name" (default: the weight's name + ".b";
// "bias": false leaves it out).  It reads whatever dtype the stream has and writes the activations'.
class LayerNorm : public Norm {
public:
    LayerNorm(const PartSpec& s, const BuildEnv& e) : Norm(e) {
        const Json* eps = s.params.find("eps");
        if (!eps || !eps->is_number()) throw ConfigError("layernorm needs 'eps'");
        eps_ = (float)eps->as_double();
        width_ = s.params.get_int("width", e.width);
        name_ = s.params.get_string("weight_name", "weight");
        has_bias_ = s.params.get_bool("bias", true);
        bias_name_ = s.params.get_string("bias_name", name_ + ".b");
        declare(name_, {width_}, false, true);
        if (has_bias_) declare(bias_name_, {width_});
    }
    Tensor forward(Ops& ops, const Tensor& x) override {
        return ops.layernorm_to(x, tensor(name_), has_bias_ ? &tensor(bias_name_) : nullptr, eps_, env.dtype);
    }
    bool layer_parts(Tensor* weight, Tensor* bias, float* eps) const override {
        *weight = tensor(name_);
        *bias = has_bias_ ? tensor(bias_name_) : Tensor();
        *eps = eps_;
        return true;
    }

private:
    float eps_;
    int64_t width_;
    bool has_bias_;
    std::string name_, bias_name_;
};

// ------------------------------------------------------------------ rotary encoding, NeoX pairing
// The pair (i, i + rotary_dim/2) of every query and key head is rotated by the angle pos / theta^(2i / rotary_dim).
// The angle is formed as the reference forms it (cuda_math_kernels.cu:337-339, cpu_ops.cpp:26-30): the denominator
// theta^(2i/d) in fp32 (powf), then one fp32 division of the position by it.  The denominators are a table of
// rotary_dim/2 numbers, made once here; the kernel divides and takes sine and cosine per row.
class RotaryNeox : public Position {
public:
    RotaryNeox(const PartSpec& s, const BuildEnv& e) : Position(e) {
        theta_ = s.params.get_double("theta", 0);
        head_dim_ = (int)s.params.get_int("head_dim", 0);
        rotary_dim_ = (int)s.params.get_int("rotary_dim", head_dim_);
        if (theta_ <= 1.0) throw ConfigError("rotary_neox: 'theta' must be greater than 1");
        if (rotary_dim_ <= 0 || rotary_dim_ % 2 || rotary_dim_ > head_dim_)
            throw ConfigError(format("rotary_neox: rotary_dim %d must be even and at most head_dim %d", rotary_dim_, head_dim_));
        table_.resize(rotary_dim_ / 2);
        for (int i = 0; i < rotary_dim_ / 2; ++i)
            table_[i] = powf((float)theta_, (2.0f * (float)i) / (float)rotary_dim_);
    }
    void finalize(Ops& ops) override {
        Position::finalize(ops);
        auto mem = std::make_shared<DeviceBuffer>(table_.size() * sizeof(float));
        cuda_check(cudaMemcpyAsync(mem->get(), table_.data(), table_.size() * sizeof(float), cudaMemcpyHostToDevice, ops.stream()),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
        denominators_ = (const float*)mem->get();
        hold(mem);
    }
    bool rotary(const float** denominators, int* rotary_dim) const override {
        *denominators = denominators_;
        *rotary_dim = rotary_dim_;
        return true;
    }
    const std::vector<float>& table() const { return table_; }

private:
    double theta_;
    int head_dim_, rotary_dim_;
    std::vector<float> table_;
    const float* denominators_ = nullptr;
};

// Leaves queries and keys as they are: not rotary, and apply() does nothing.
class NoPosition : public Position {
public:
    NoPosition(const PartSpec&, const BuildEnv& e) : Position(e) {}
};

// ------------------------------------------------------------------ rotary encoding, neighbouring pairs
// Neighbours (2i, 2i + 1) among the first `dims` numbers of a head turn by the angle pos * w_i, w_i = base^(-2i / dims).
// "scaling" {factor, original, fast, slow} stretches the long wavelengths: a pair that completes t turns within
// `original` positions has index d(t) = dims * ln(original / (2 pi t)) / (2 ln base); pairs up to index
// first = max(floor(d(fast)), 0) keep their w_i, pairs from last = min(ceil(d(slow)), dims - 1) on turn `factor` times
// slower, and between the two the mix moves linearly, mix_i = clamp((i - first) / max(last - first, 0.001), 0, 1):
// w_i <- (1 - mix_i) w_i + mix_i w_i / factor.  Cosine and sine are then multiplied by 1 + 0.1 ln(factor).
// The table is made once on the host in double precision and rounded to fp32; the angle is fp32(pos) * w_i in the kernel.
class RotaryPairs : public Position {
public:
    RotaryPairs(const PartSpec& s, const BuildEnv& e) : Position(e) {
        const double base = s.params.get_double("base", 0);
        dims_ = (int)s.params.get_int("dims", 0);
        // "layout": "neighbours" pairs (2i, 2i + 1); "halves" pairs (i, i + dims / 2); the table is the same
        const std::string layout = s.params.get_string("layout", "neighbours");
        if (layout != "neighbours" && layout != "halves") throw ConfigError("rotary_pairs: 'layout' is \"neighbours\" or \"halves\"");
        halves_ = layout == "halves";
        if (base <= 1.0) throw ConfigError("rotary_pairs: 'base' must be greater than 1");
        if (dims_ <= 0 || dims_ % 2) throw ConfigError(format("rotary_pairs: 'dims' = %d must be even and positive", dims_));
        const int half = dims_ / 2;
        table_.resize(half);
        std::vector<double> f(half);
        for (int i = 0; i < half; ++i) f[i] = pow(base, -2.0 * i / dims_);
        const Json* sc = s.params.find("scaling");
        if (sc && sc->is_object()) {
            const double factor = sc->get_double("factor", 1.0), original = sc->get_double("original", 0);
            const double fast = sc->get_double("fast", 32.0), slow = sc->get_double("slow", 1.0);
            if (!(factor > 0) || !(original > 0) || !(fast > 0) || !(slow > 0))
                throw ConfigError("rotary_pairs: 'scaling' needs positive factor, original, fast and slow");
            auto dim_of = [&](double turns) { return dims_ * log(original / (2.0 * M_PI * turns)) / (2.0 * log(base)); };
            const double first = std::max(floor(dim_of(fast)), 0.0), last = std::min(ceil(dim_of(slow)), (double)dims_ - 1.0);
            for (int i = 0; i < half; ++i) {
                double mix = ((double)i - first) / std::max(last - first, 0.001);
                mix = mix < 0 ? 0 : (mix > 1 ? 1 : mix);
                f[i] = f[i] / factor * mix + f[i] * (1.0 - mix);
            }
            mult_ = (float)(0.1 * log(factor) + 1.0);
        }
        for (int i = 0; i < half; ++i) table_[i] = (float)f[i];
    }
    void finalize(Ops& ops) override {
        Position::finalize(ops);
        auto mem = std::make_shared<DeviceBuffer>(table_.size() * sizeof(float));
        cuda_check(cudaMemcpyAsync(mem->get(), table_.data(), table_.size() * sizeof(float), cudaMemcpyHostToDevice, ops.stream()),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
        freq_ = (const float*)mem->get();
        hold(mem);
    }
    bool pairs(const float** frequencies, float* multiplier, int* dims) const override {
        if (halves_) return false;
        *frequencies = freq_;
        *multiplier = mult_;
        *dims = dims_;
        return true;
    }
    bool halves(const float** frequencies, float* multiplier, int* dims) const override {
        if (!halves_) return false;
        *frequencies = freq_;
        *multiplier = mult_;
        *dims = dims_;
        return true;
    }
    const std::vector<float>& table() const { return table_; }
    // inside a stacked q/k/v buffer: every query and key head's first `dims` dimensions
    void apply(Ops& ops, Tensor& qkv, const StepContext& ctx, int n_heads, int n_kv_heads, int head_dim) override {
        if (halves_) throw ConfigError("rotary_pairs: the halves layout is applied by the mixers that ask for it, not inside a stacked q/k/v buffer");
        if (dims_ > head_dim) throw ConfigError(format("rotary_pairs: %d rotated dimensions in heads of %d", dims_, head_dim));
        ops.rotate_pairs(qkv, ctx, freq_, mult_, n_heads + n_kv_heads, head_dim, 0, dims_);
    }

private:
    int dims_;
    bool halves_ = false;
    float mult_ = 1.0f;
    std::vector<float> table_;
    const float* freq_ = nullptr;
};

// ------------------------------------------------------------------ grouped-query attention over the paged cache
// q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (one product over the stacked matrices); q and k are encoded with the
// position part; k and v go to the cache at each row's (sequence, position); every query attends to the keys of its
// sequence up to its own position, or to the last `window` of them; the result goes through Wo and the residual is
// added in that product's epilogue.
//
// Reference order of operations: transformer.cpp:1013-1059 (norm is the block's), q/k/v bias in the product's
// epilogue (hpc_k_quants.cu:422-437), rotation and cache write in one kernel (cuda_math_kernels.cu:363-404),
// grouped heads h -> h / (heads / kv heads) and 1/sqrt(head_dim) scaling (attention_kernels.cu:45,
// cpu_ops.cpp:49-53), the output product with the residual (transformer.cpp:1057-1059).
class GQAttention : public Mixer {
public:
    GQAttention(const PartSpec& s, const BuildEnv& e) : Mixer(e) {
        nq_ = (int)s.params.get_int("n_heads", 0);
        nkv_ = (int)s.params.get_int("n_kv_heads", nq_);
        hd_ = (int)s.params.get_int("head_dim", 0);
        vd_ = (int)s.params.get_int("v_head_dim", hd_);              // values may have a size of their own
        if (nq_ <= 0 || nkv_ <= 0 || hd_ <= 0 || vd_ <= 0) throw ConfigError("gqa_attention needs n_heads, n_kv_heads and head_dim");
        if (nq_ % nkv_) throw ConfigError(format("%d heads cannot share %d key/value heads", nq_, nkv_));
        window_ = (int)s.params.get_int("window", 0);
        keep_first_ = (int)s.params.get_int("keep_first", 0);         // behind a window, positions below this stay visible
        if (keep_first_ < 0) throw ConfigError("gqa_attention: 'keep_first' must not be negative");
        scale_ = (float)s.params.get_double("scale", 1.0 / sqrt((double)hd_));
        qkv_bias_ = s.params.get_bool("qkv_bias", true);
        out_bias_ = s.params.get_bool("out_bias", false);
        position_ = adopt("", build<Position>("position", s.part("position"), e));
        const int64_t qd = (int64_t)nq_ * hd_, kvd = (int64_t)nkv_ * hd_, vvd = (int64_t)nkv_ * vd_, w = e.width;
        // Heads that talk: "distance_slope_base" b > 0 takes 2^(-b (h + 1) / heads) * (i - j) off head h's score; "talk" names
        // a tensor [heads, heads] that mixes the heads' scores before the softmax; "gate" names a projection [heads * v, width]
        // whose sigmoid multiplies the heads' results element by element (it reads the mixer's input, like q, k and v);
        // "value_mix": "first" leaves this layer's values for later layers of the pass under "value_mix_key", "blend" replaces
        // v by (1 - lambda) v + lambda v_first before it is cached, lambda being the tensor "value_mix_weight".
        slope_base_ = s.params.get_double("distance_slope_base", 0.0);
        talk_name_ = s.params.get_string("talk", "");
        gate_name_ = s.params.get_string("gate", "");
        value_mix_ = s.params.get_string("value_mix", "");
        value_key_ = s.params.get_string("value_mix_key", "values.first");
        lambda_name_ = s.params.get_string("value_mix_weight", "vmix");
        if (!value_mix_.empty() && value_mix_ != "first" && value_mix_ != "blend")
            throw ConfigError("gqa_attention: 'value_mix' is \"first\", \"blend\" or absent");
        talking_ = slope_base_ > 0.0 || !talk_name_.empty() || !gate_name_.empty() || !value_mix_.empty();
        const int64_t gd = gate_name_.empty() ? 0 : (int64_t)nq_ * vd_;
        declare_stacked("w_qkv", qd + kvd + vvd + gd, w);
        if (qkv_bias_) declare_stacked("b_qkv", qd + kvd + vvd + gd, 1);      // a vector: one column, members under one another
        // tensor names: Hugging Face's unless the specification gives others ("names": {"q": ..., "k": ..., "v": ..., "o": ...})
        const Json* names = s.params.find("names");
        const char* roles[4] = {"q", "k", "v", "o"};
        const char* defaults[4] = {"q_proj", "k_proj", "v_proj", "o_proj"};
        std::string stem[4];
        bool bare = false;
        for (int i = 0; i < 4; ++i) {
            stem[i] = defaults[i];
            if (names && names->is_object() && names->has(roles[i])) {
                stem[i] = names->at(roles[i]).as_string();
                bare = true;
            }
        }
        const std::string wsuf = bare ? "" : ".weight", bsuf = s.params.get_string("bias_suffix", ".bias");
        const int64_t rows[3] = {qd, kvd, vvd}, first[3] = {0, qd, qd + kvd};
        for (int i = 0; i < 3; ++i) {
            declare(stem[i] + wsuf, {rows[i], w}).stack("w_qkv", first[i]);
            if (qkv_bias_) declare(stem[i] + bsuf, {rows[i]}).stack("b_qkv", first[i]);
        }
        o_name_ = stem[3] + wsuf;
        o_bias_name_ = stem[3] + bsuf;
        declare(o_name_, {w, (int64_t)nq_ * vd_});
        if (out_bias_) declare(o_bias_name_, {w});
        if (gd) declare(gate_name_, {gd, w}).stack("w_qkv", qd + kvd + vvd);      // its rows of the bias stay zero
        if (!talk_name_.empty()) declare(talk_name_, {(int64_t)nq_, (int64_t)nq_});
        if (value_mix_ == "blend") declare(lambda_name_, {});
        if (talking_ && keep_first_ > 0) throw ConfigError("gqa_attention: kept first keys with talking heads are not built");
    }
    CacheRequest cache_request() const override { return CacheRequest::kv(nkv_, hd_, window_, vd_, keep_first_); }
    void finalize(Ops& ops) override {
        Mixer::finalize(ops);
        if (slope_base_ <= 0.0) return;
        std::vector<float> table((size_t)nq_);
        for (int h = 0; h < nq_; ++h) table[(size_t)h] = (float)pow(2.0, -slope_base_ * (double)(h + 1) / (double)nq_);
        auto mem = std::make_shared<DeviceBuffer>(table.size() * sizeof(float));
        cuda_check(cudaMemcpyAsync(mem->get(), table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice, ops.stream()),
                   "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
        slopes_ = (const float*)mem->get();
        hold(mem);
    }

    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view,
                    Norm* then) override {
        const Tensor& w_qkv = tensor("w_qkv");
        Tensor bias_flat;
        const Tensor* b_qkv = nullptr;
        if (qkv_bias_) {
            const Tensor& b = tensor("b_qkv");
            bias_flat = Tensor::make(b.data, b.dtype, {b.numel()});
            b_qkv = &bias_flat;
        }
        const float* denominators = nullptr;
        int rotary_dim = 0;
        Tensor qkv;
        if (talking_) return talking(ops, h, residual, ctx, view, w_qkv, b_qkv);
        if (position_->rotary(&denominators, &rotary_dim)) {
            if (vd_ != hd_) throw ConfigError("gqa_attention: a rotary encoding with values of another size than the keys is not built");
            qkv = ops.qkv_rope_write(h, w_qkv, b_qkv, ctx.row_seq, ctx.row_pos, denominators, rotary_dim, nq_, nkv_, hd_, &view);
        } else {                                    // another encoding: it changes q and k itself
            qkv = ops.linear(h, w_qkv, b_qkv);
            position_->apply(ops, qkv, ctx, nq_, nkv_, hd_);
            if (view.write) {
                if (vd_ == hd_) ops.rope_kv_write(qkv, ctx.row_seq, ctx.row_pos, nullptr, 0, nq_, nkv_, hd_, &view);
                else ops.kv_store(qkv, (int64_t)nq_ * hd_, (int64_t)(nq_ + nkv_) * hd_, view, ctx);
            }
        }
        Tensor mixed = ops.alloc(qkv.dtype, qkv.rows(), (int64_t)nq_ * vd_);
        ops.attention(qkv, qkv.ld, mixed, view, ctx, nq_, nkv_, hd_, window_, scale_);
        const Tensor& w_o = tensor(o_name_);
        const Tensor* b_o = out_bias_ ? &tensor(o_bias_name_) : nullptr;
        Tensor nw;
        float eps;
        if (then && out_scale == 1.0f && residual.dtype == mixed.dtype && then->as_rmsnorm(&nw, &eps)) {
            auto r = ops.linear_norm(Rows(mixed), w_o, nw, eps, b_o, &residual);
            return PartOut(r.first, r.second);
        }
        return PartOut(ops.linear_residual(Rows(mixed), w_o, b_o, residual, out_scale));
    }

private:
    // The talking form: one product for q, k, v and the gate; the position part may change q and k; keys and (blended) values
    // go to the cache; scores of all heads, mixed, through the softmax and the values; gate; output product.
    PartOut talking(Ops& ops, const Rows& h, const Tensor& residual, const StepContext& ctx, const CacheView& view, const Tensor& w_qkv,
                    const Tensor* b_qkv) {
        const float* denominators = nullptr;
        int rotary_dim = 0;
        if (position_->rotary(&denominators, &rotary_dim)) throw ConfigError("gqa_attention: talking heads with a rotary table in the product are not built");
        Tensor qkv = ops.linear(h, w_qkv, b_qkv);
        position_->apply(ops, qkv, ctx, nq_, nkv_, hd_);
        Ops::TalkSpec sp;
        sp.heads = nq_;
        sp.kv_heads = nkv_;
        sp.dim = hd_;
        sp.vdim = vd_;
        sp.window = window_;
        sp.scale = scale_;
        sp.slopes = slopes_;
        sp.talk = talk_name_.empty() ? nullptr : &tensor(talk_name_);
        sp.q_off = 0;
        sp.k_off = (int64_t)nq_ * hd_;
        sp.v_off = sp.k_off + (int64_t)nkv_ * hd_;
        sp.gate_off = gate_name_.empty() ? -1 : sp.v_off + (int64_t)nkv_ * vd_;
        const Tensor* blend = nullptr;
        Tensor kept;
        Tensor* keep = nullptr;
        if (!value_mix_.empty()) {
            if (!ctx.values) throw KernelError("gqa_attention: blending values needs the pass's shared rows");
            if (value_mix_ == "first") {
                if (ctx.values->rows.count(value_key_)) throw ConfigError("two layers leave their values under '" + value_key_ + "'");
                kept = Tensor::make(ctx.values->arena->alloc((size_t)qkv.rows() * nkv_ * vd_ * dtype_size(qkv.dtype)), qkv.dtype,
                                    {qkv.rows(), (int64_t)nkv_ * vd_});
                keep = &kept;
            } else {
                auto it = ctx.values->rows.find(value_key_);
                if (it == ctx.values->rows.end()) throw ConfigError("no earlier layer left values under '" + value_key_ + "' to blend with");
                blend = &it->second;
            }
        }
        ops.talk_store(qkv, sp, view, ctx, blend, blend ? &tensor(lambda_name_) : nullptr, keep);
        if (keep) ctx.values->rows[value_key_] = kept;
        Tensor mixed = ops.talk_attention(qkv, sp, view, ctx);
        const Tensor& w_o = tensor(o_name_);
        const Tensor* b_o = out_bias_ ? &tensor(o_bias_name_) : nullptr;
        if (!residual.defined()) {                  // the block sums itself: the result alone, 32-bit
            Tensor y = ops.linear(Rows(mixed), w_o, b_o, nullptr, (int)DType::F32);
            if (out_scale != 1.0f) ops.scale_rows(y, out_scale);
            return PartOut(y);
        }
        return PartOut(ops.linear_residual(Rows(mixed), w_o, b_o, residual, out_scale));
    }

    int nq_, nkv_, hd_, vd_, window_, keep_first_;
    float scale_;
    bool qkv_bias_, out_bias_;
    Position* position_;
    std::string o_name_, o_bias_name_;
    double slope_base_ = 0.0;
    bool talking_ = false;
    std::string talk_name_, gate_name_, value_mix_, value_key_, lambda_name_;
    const float* slopes_ = nullptr;
};

// ------------------------------------------------------------------ gated feed-forward: x + Wd (silu(Wg h) * (Wu h))
// Gate and up are one product, as the reference runs the two in one launch (transformer.cpp:1064-1066): their rows
// are stacked alternately (gate 0, up 0, gate 1, ...), so that every tile of the product holds both halves of a
// pair and silu(z) = z / (1 + e^-z) times up (cpu_ops.cpp:85-101, without its shortcuts for |z| > 20) can be
// applied in the product's epilogue; the residual is added in the down product's epilogue (transformer.cpp:1072).
class SwiGLU : public FeedForward {
public:
    SwiGLU(const PartSpec& s, const BuildEnv& e) : FeedForward(e) {
        inner_ = s.params.get_int("inner", 0);
        if (inner_ <= 0) throw ConfigError("swiglu needs 'inner'");
        // tensor names: Hugging Face's unless the specification gives others ("names": {"gate": ..., "up": ..., "down": ...})
        const Json* names = s.params.find("names");
        auto name_of = [&](const char* role, const char* fallback) {
            return names && names->is_object() && names->has(role) ? names->at(role).as_string() : std::string(fallback);
        };
        down_ = name_of("down", "down_proj.weight");
        // "activation" of the gate: "silu" (default) or "gelu_tanh"
        const std::string act = s.params.get_string("activation", "silu");
        if (act != "silu" && act != "gelu_tanh") throw ConfigError("swiglu: activation '" + act + "' is not one it has (silu, gelu_tanh)");
        act_ = act == "gelu_tanh" ? 2 : 1;
        declare_stacked("w_gate_up", 2 * inner_, e.width);
        declare(name_of("gate", "gate_proj.weight"), {inner_, e.width}).stack("w_gate_up", 0, 2);
        declare(name_of("up", "up_proj.weight"), {inner_, e.width}).stack("w_gate_up", 1, 2);
        declare(down_, {e.width, inner_});
    }
    PartOut forward(Ops& ops, const Rows& h, const Tensor& residual, const StepContext&, Norm* then) override {
        Tensor inner = ops.linear_swiglu(h, tensor("w_gate_up"), act_);
        Tensor nw;
        float eps;
        if (then && residual.dtype == inner.dtype && then->as_rmsnorm(&nw, &eps)) {
            auto r = ops.linear_norm(Rows(inner), tensor(down_), nw, eps, nullptr, &residual);
            return PartOut(r.first, r.second);
        }
        // a 32-bit stream beside 16-bit activations: the product's result stays 32-bit and is added there
        return PartOut(ops.linear_residual(Rows(inner), tensor(down_), nullptr, residual));
    }

private:
    int64_t inner_;
    int act_ = 1;
    std::string down_;
};

// ------------------------------------------------------------------ pre-norm residual block
// x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)); x = token_input(x) (the last two if the block has them).  The sums happen inside the mixer's and the
// feed-forward's last product (each gets the residual stream and returns it with its own output added), as in the
// reference (transformer.cpp:997-1074).  Which mixer, feed-forward and norms a block has is its specification's.
class PreNormBlock : public Block {
public:
    PreNormBlock(const PartSpec& s, const BuildEnv& e) : Block(e) {
        const PartSpec& n1 = s.part("norm1");
        const PartSpec& mx = s.part("mixer");
        norm1_ = adopt(n1.prefix, build<Norm>("norm", n1, e));
        mixer_ = adopt(mx.prefix, build<Mixer>("mixer", mx, e));
        // a block may go without a feed-forward (then it has no second norm either), and may end with a token input
        if (s.parts.count("feed_forward")) {
            const PartSpec& n2 = s.part("norm2");
            const PartSpec& ff = s.part("feed_forward");
            norm2_ = adopt(n2.prefix, build<Norm>("norm", n2, e));
            ffn_ = adopt(ff.prefix, build<FeedForward>("feed_forward", ff, e));
        }
        if (s.parts.count("token_input")) {
            const PartSpec& ti = s.part("token_input");
            token_input_ = adopt(ti.prefix, build<TokenInput>("token_input", ti, e));
        }
        // "input_conv": {"taps": n, "mixer": name, "feed_forward": name}: what each sublayer reads, h = norm(x), becomes
        // h + conv(h), a causal convolution over time on each channel with the tensor [width, n] of that name (no bias),
        // zeros before a sequence's start; the last n - 1 rows h of each sublayer are kept per sequence beside what the mixer
        // asks of the cache.  The norms are layer norms; norm and convolution run as one kernel.
        const Json* ic = s.params.find("input_conv");
        if (ic && ic->is_object()) {
            taps_ = (int)ic->get_int("taps", 0);
            if (taps_ < 1 || taps_ > 8) throw ConfigError("prenorm block: 'input_conv' needs 1 to 8 'taps'");
            conv1_ = ic->get_string("mixer", "");
            conv2_ = ffn_ ? ic->get_string("feed_forward", "") : "";
            if (conv1_.empty() || (ffn_ && conv2_.empty())) throw ConfigError("prenorm block: 'input_conv' names a tensor for every sublayer");
            declare(conv1_, {e.width, (int64_t)taps_});
            if (ffn_) declare(conv2_, {e.width, (int64_t)taps_});
        }
    }
    CacheRequest cache_request() const override {
        if (taps_ == 0) return mixer_->cache_request();
        std::vector<CacheRequest> all{mixer_->cache_request()};
        const int64_t hist = std::max<int64_t>(1, (int64_t)(taps_ - 1) * env.width);
        all.push_back(CacheRequest::state({hist}, DType::F32));
        if (ffn_) all.push_back(CacheRequest::state({hist}, DType::F32));
        return CacheRequest::flat(all);
    }
    Norm* first_norm() override { return taps_ ? nullptr : norm1_; }        // with a convolution the norm runs inside this block

    PartOut forward(Ops& ops, const Tensor& x, const Rows* normed, const StepContext& ctx, const CacheView& view,
                    Norm* then) override {
        if (taps_) return forward_conv(ops, x, ctx, view, then);
        Rows h = normed ? *normed : Rows(norm1_->forward(ops, x));
        Norm* after_last = token_input_ ? nullptr : then;       // a token input changes the stream after the last product
        PartOut b = mixer_->forward(ops, h, x, ctx, view, ffn_ ? norm2_ : after_last);
        if (ffn_) {
            Rows h2 = b.has_normed ? b.normed : Rows(norm2_->forward(ops, b.x));
            const Tensor mixed = b.x;
            b = ffn_->forward(ops, h2, mixed, ctx, after_last);
        }
        if (token_input_) {
            token_input_->forward(ops, b.x, ctx);
            b.has_normed = false;
        }
        if (then && !b.has_normed) {
            b.normed = Rows(then->forward(ops, b.x));
            b.has_normed = true;
        }
        return b;
    }

private:
    // the same block with h + conv(h) ahead of every sublayer
    PartOut forward_conv(Ops& ops, const Tensor& x, const StepContext& ctx, const CacheView& view, Norm* then) {
        if (x.dtype != DType::F32) throw ConfigError("prenorm block: an input convolution needs a 32-bit residual stream");
        const CacheRequest mixer_request = mixer_->cache_request();
        const size_t n_mixer = mixer_request.kind == CacheRequest::None ? 1 : CacheRequest::flat_size(mixer_request);
        if (view.kind != CacheRequest::Several || view.parts.size() != n_mixer + (ffn_ ? 2 : 1))
            throw KernelError("prenorm block: the cache view does not have the mixer's parts and the convolutions' histories");
        Tensor w, b;
        float eps = 0.f;
        if (!norm1_->layer_parts(&w, &b, &eps)) throw ConfigError("prenorm block: an input convolution follows a layer norm");
        Rows h(ops.norm_conv(x, w, b.defined() ? &b : nullptr, eps, tensor(conv1_), view.parts[n_mixer], ctx, env.dtype));
        static const CacheView none;
        PartOut out = mixer_->forward(ops, h, x, ctx, mixer_request.kind == CacheRequest::None ? none : view.member(0, mixer_request), nullptr);
        if (ffn_) {
            if (!norm2_->layer_parts(&w, &b, &eps)) throw ConfigError("prenorm block: an input convolution follows a layer norm");
            Rows h2(ops.norm_conv(out.x, w, b.defined() ? &b : nullptr, eps, tensor(conv2_), view.parts[n_mixer + 1], ctx, env.dtype));
            const Tensor mixed = out.x;
            out = ffn_->forward(ops, h2, mixed, ctx, nullptr);
        }
        if (token_input_) token_input_->forward(ops, out.x, ctx);
        out.has_normed = false;
        if (then) {
            out.normed = Rows(then->forward(ops, out.x));
            out.has_normed = true;
        }
        return out;
    }

    Norm *norm1_ = nullptr, *norm2_ = nullptr;
    Mixer* mixer_ = nullptr;
    FeedForward* ffn_ = nullptr;
    TokenInput* token_input_ = nullptr;
    int taps_ = 0;
    std::string conv1_, conv2_;
};

namespace {
PartRegistrar r1("norm", "rmsnorm", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RMSNorm(s, e); });
PartRegistrar r1b("norm", "layernorm", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new LayerNorm(s, e); });
PartRegistrar r2b("position", "rotary_pairs", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RotaryPairs(s, e); });
PartRegistrar r2("position", "rotary_neox", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new RotaryNeox(s, e); });
PartRegistrar r3("position", "none", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new NoPosition(s, e); });
PartRegistrar r4("mixer", "gqa_attention", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new GQAttention(s, e); });
PartRegistrar r5("feed_forward", "swiglu", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new SwiGLU(s, e); });
PartRegistrar r6("block", "prenorm", [](const PartSpec& s, const BuildEnv& e) -> Part* { return new PreNormBlock(s, e); });
}  // namespace

}  // namespace friday
