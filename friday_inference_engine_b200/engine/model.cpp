// DecoderModel: parts from a specification, weights from a source, one pass over rows (model.h).
#include "friday/model.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <set>

namespace friday {

// FRIDAY_DUMP_LAYERS=<folder>: the residual stream after every program entry of every pass is written there as
// little-endian fp32 [rows, width] (pass<k>_entry<i>.f32), for comparing a model layer by layer with another
// implementation.  It waits for the device after every layer: for debugging only.
static void dump_stream(Ops& ops, const Tensor& x, int pass, size_t entry) {
    const char* dir = getenv("FRIDAY_DUMP_LAYERS");
    if (!dir || !dir[0]) return;
    std::vector<float> host((size_t)x.numel());
    if (x.dtype == DType::F32) {
        cuda_check(cudaMemcpyAsync(host.data(), x.data, x.bytes(), cudaMemcpyDeviceToHost, ops.stream()), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
    } else {
        std::vector<uint16_t> raw((size_t)x.numel());
        cuda_check(cudaMemcpyAsync(raw.data(), x.data, x.bytes(), cudaMemcpyDeviceToHost, ops.stream()), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
        for (size_t i = 0; i < raw.size(); ++i) {
            const uint32_t bits = (uint32_t)raw[i] << 16;
            memcpy(&host[i], &bits, 4);
        }
    }
    const std::string path = format("%s/pass%d_entry%zu.f32", dir, pass, entry);
    if (FILE* f = fopen(path.c_str(), "wb")) {
        fwrite(host.data(), sizeof(float), host.size(), f);
        fclose(f);
    }
}

class DecoderModel::Root : public Part {
public:
    explicit Root(const BuildEnv& e) : Part(e) {}
};

DecoderModel::DecoderModel(const ModelSpec& s, DType dtype) : spec(s) {
    env.width = s.width;
    env.dtype = dtype;
    if (s.vocab_size <= 0 || s.width <= 0) throw ConfigError("a model needs a vocabulary and a width");
    owners = spec.cache_entries();
    for (const auto& ls : spec.layers) layers.emplace_back(build<Block>("block", ls, env));
    final_norm.reset(build<Norm>("norm", spec.final_norm, env));
    if (!spec.embed_norm.kind.empty()) embed_norm.reset(build<Norm>("norm", spec.embed_norm, env));
    for (const auto& c : spec.program)
        if (c.inject >= (int)spec.injections.size()) throw ConfigError("a program entry names an injection that the model does not have");
    root_.reset(new Root(env));
    for (const auto& inj : spec.injections) root_->declare(inj.weight, {spec.width, 2 * spec.width});
    for (const auto& sh : spec.shared) root_->declare(sh.first, sh.second);
    root_->declare(spec.embedding, {spec.vocab_size, spec.width});
    if (!spec.position_table.empty()) {
        if (!spec.residual_f32 || !spec.embed_norm.kind.empty() || spec.embed_scale != 1.0)
            throw ConfigError("a learned position table is added to plain token rows of a 32-bit residual stream");
        root_->declare(spec.position_table, {spec.max_positions, spec.width});
    }
    if (spec.has_embed_state()) {
        const ModelSpec::PairTable& pt = spec.pair_table;
        if (!spec.residual_f32 || !spec.embed_norm.kind.empty() || spec.embed_scale != 1.0 || !spec.position_table.empty())
            throw ConfigError("a token-pair table is added to plain token rows of a 32-bit residual stream");
        if (pt.buckets <= 0 || pt.mul_prev < 0 || pt.mul_cur < 0) throw ConfigError("a token-pair table needs positive 'buckets' and multipliers that are not negative");
        root_->declare(pt.table, {pt.buckets + 1, spec.width});
    }
    if (!spec.head.empty()) root_->declare(spec.head, {spec.vocab_size, spec.width});
    if (!spec.head_bias.empty()) root_->declare(spec.head_bias, {spec.vocab_size});
}

std::vector<Part::Named> DecoderModel::named_params() {
    std::vector<Part::Named> out;
    root_->named_params("", out);
    for (size_t i = 0; i < layers.size(); ++i) layers[i]->named_params(spec.layers[i].prefix, out);
    final_norm->named_params(spec.final_norm.prefix, out);
    if (embed_norm) embed_norm->named_params(spec.embed_norm.prefix, out);
    return out;
}

std::map<int, CacheRequest> DecoderModel::cache_requests() const {
    std::map<int, CacheRequest> out;
    for (const auto& kv : owners) out[kv.first] = layers[spec.program[kv.second].layer]->cache_request();
    if (spec.has_embed_state()) {
        if (out.count(ModelSpec::kEmbedStateEntry)) throw ConfigError("a program entry uses the cache entry that the embedding's state takes");
        out[ModelSpec::kEmbedStateEntry] = CacheRequest::state({1}, DType::I32);      // the previous token
    }
    return out;
}

static DType storage_dtype(const StoredTensor& st, const ParamDecl& d, DType compute, const std::string& name) {
    if (d.integer) return DType::I32;
    if (!stored_dtype_is_float(st.dtype))
        throw WeightsError("tensor '" + name + "': an integer tensor (" + st.dtype + ") where a floating one is needed");
    if (compute == DType::F32 || stored_dtype_is_32bit_float(st.dtype)) return DType::F32;
    return compute;
}

std::vector<StoredParam> plan_storage(const std::vector<Part::Named>& all, const WeightSource& source, DType compute,
                                      const std::vector<std::string>& ignorable) {
    std::vector<Part::Named> named;
    std::set<std::string> seen;
    for (auto& e : all)
        if (seen.insert(e.name).second) named.push_back(e);
    check_names(named, source, ignorable);
    std::vector<StoredParam> plan;
    // a stacked tensor is 32-bit if any member is stored so
    std::map<std::pair<Part*, std::string>, DType> stacked_dtype;
    for (const auto& e : named) {
        StoredTensor st;
        source.info(e.name, &st);
        StoredParam s;
        s.param = e;
        s.param.decl.shape = st.shape;          // equal but for sizes left to the checkpoint (-1), which it gives here
        s.dtype = storage_dtype(st, e.decl, compute, e.name);
        if (!e.decl.into.empty()) {
            auto key = std::make_pair(e.owner, e.decl.into);
            auto it = stacked_dtype.find(key);
            if (it == stacked_dtype.end()) stacked_dtype[key] = s.dtype;
            else if (s.dtype == DType::F32) it->second = DType::F32;
        }
        plan.push_back(s);
    }
    for (auto& s : plan)
        if (!s.param.decl.into.empty()) s.dtype = stacked_dtype[std::make_pair(s.param.owner, s.param.decl.into)];
    return plan;
}

size_t load_params(const std::vector<StoredParam>& plan, WeightSource& source, Ops& ops) {
    size_t bytes = 0;
    for (const auto& s : plan) {          // stacked tensors first
        const Part::Named& e = s.param;
        if (e.decl.into.empty() || e.owner->tensors.count(e.decl.into)) continue;
        const std::vector<int64_t>* shape = nullptr;
        for (const auto& st : e.owner->stacked)
            if (st.first == e.decl.into) shape = &st.second;
        if (!shape) throw ConfigError("a parameter is stacked into '" + e.decl.into + "', which its part never declared");
        // zeroed: a stacked tensor may have rows that no parameter fills (the bias of a member that has none)
        auto mem = std::make_shared<DeviceBuffer>((size_t)(*shape)[0] * (*shape)[1] * dtype_size(s.dtype), true);
        e.owner->set_tensor(e.decl.into, Tensor::make(mem->get(), s.dtype, *shape));
        e.owner->hold(mem);
        bytes += mem->bytes();
    }
    for (const auto& s : plan) {
        const Part::Named& e = s.param;
        Tensor dst;
        const int64_t cols = e.decl.shape.size() >= 2 ? e.decl.shape.back() : 1;
        if (e.decl.into.empty()) {
            int64_t n = 1;
            for (int64_t d : e.decl.shape) n *= d;
            auto mem = std::make_shared<DeviceBuffer>((size_t)n * dtype_size(s.dtype));
            Tensor t = Tensor::make(mem->get(), s.dtype, e.decl.shape);
            e.owner->set_tensor(e.local, t);
            e.owner->hold(mem);
            bytes += mem->bytes();
            dst = t;
            dst.ld = cols;
        } else if (e.decl.col0 >= 0) {           // side by side: its own columns of the rows from row0 on
            const Tensor& big = e.owner->tensor(e.decl.into);
            if (e.decl.col0 + cols > big.cols())
                throw ConfigError("parameter '" + e.name + "' does not fit the columns of '" + e.decl.into + "' that it is stacked into");
            dst = big;
            dst.data = (char*)big.data + ((size_t)e.decl.row0 * big.ld + (size_t)e.decl.col0) * dtype_size(big.dtype);
            dst.ld = big.ld;
        } else {
            const Tensor& big = e.owner->tensor(e.decl.into);
            if (big.cols() != cols)
                throw ConfigError("parameter '" + e.name + "' does not have the columns of '" + e.decl.into + "' that it is stacked into");
            dst = big;
            dst.data = (char*)big.data + (size_t)e.decl.row0 * big.ld * dtype_size(big.dtype);
            dst.ld = big.ld * e.decl.row_step;
        }
        source.load(e.name, dst, ops.stream());
    }
    cuda_check(cudaStreamSynchronize(ops.stream()), "cudaStreamSynchronize");
    return bytes;
}

std::vector<StoredParam> DecoderModel::plan_storage(const WeightSource& source) {
    return friday::plan_storage(named_params(), source, env.dtype, spec.ignorable);
}

void DecoderModel::load(WeightSource& source, Ops& ops) {
    parameter_bytes_ = load_params(plan_storage(source), source, ops);
    embedding = root_->tensor(spec.embedding);
    head = spec.head.empty() ? embedding : root_->tensor(spec.head);       // tied: one copy in memory
    if (!spec.head_bias.empty()) head_bias = root_->tensor(spec.head_bias);
    if (!spec.position_table.empty()) position_table = root_->tensor(spec.position_table);
    if (spec.has_embed_state()) pair_table = root_->tensor(spec.pair_table.table);
    injections.clear();
    for (const auto& inj : spec.injections) injections.push_back(root_->tensor(inj.weight));
    std::map<std::string, Tensor> shared;
    for (const auto& sh : spec.shared) shared[sh.first] = root_->tensor(sh.first);
    for (auto& l : layers) {
        l->bind_shared(shared);
        l->finalize(ops);
    }
    final_norm->finalize(ops);
    if (embed_norm) embed_norm->finalize(ops);
}

DecoderModel::RunOut DecoderModel::run(Ops& ops, const StepContext& ctx, const std::vector<CacheView>& views,
                                       bool with_final_norm, Arena* layer_arenas[2]) {
    Arena* outer = ops.arena;
    Tensor x;
    PassValues values;                      // what layers leave for later layers lives in the caller's arena
    values.arena = outer;
    StepContext with_values = ctx;
    with_values.values = &values;
    if (pair_table.defined()) {
        if (views.size() != spec.program.size() + 1) throw KernelError("the model's embedding keeps a state and was given no view of it");
        const ModelSpec::PairTable& pt = spec.pair_table;
        x = ops.embed_pair_rows(ctx, embedding, pair_table, pt.buckets, pt.mul_prev, pt.mul_cur, views.back());
    } else if (position_table.defined()) {
        x = ops.embed_pos_rows(ctx, embedding, position_table);
    } else if (spec.residual_f32 && !embed_norm) {
        x = ops.embed_rows(ctx.tokens, ctx.rows, embedding, (float)spec.embed_scale);      // no rounding between table and stream
    } else {
        x = ops.embedding(ctx.tokens, ctx.rows, embedding);
        if (spec.embed_scale != 1.0) ops.scale_rows(x, (float)spec.embed_scale);
        if (embed_norm) x = embed_norm->forward(ops, x);
    }
    if (spec.residual_f32 && x.dtype != DType::F32)
        throw ConfigError("a model with a 32-bit residual stream needs an embedding norm (or a token table) that yields 32-bit rows");
    const Tensor x0 = x;                    // what injections feed back in; it lives in the caller's arena
    Rows normed;
    bool has_normed = false;
    const size_t n = spec.program.size();
    static int passes = 0;
    const bool dumping = getenv("FRIDAY_DUMP_LAYERS") != nullptr;
    const int pass_no = dumping ? passes++ : 0;
    for (size_t i = 0; i < n; ++i) {
        const LayerCall& call = spec.program[i];
        Block* block = layers[call.layer].get();
        // the last entry's results must outlive the loop: they come from the caller's arena
        Arena* mine = (i + 1 == n) ? outer : layer_arenas[i & 1];
        if (mine != outer) mine->reset();
        ops.arena = mine;
        if (call.inject >= 0) {
            // x <- W [x; x0]: both halves in the activation dtype, the sum of products straight into the stream's dtype
            Tensor both = ops.concat_cast(x, x0, env.dtype);
            x = ops.linear(Rows(both), injections[(size_t)call.inject], nullptr, nullptr, (int)x.dtype);
            has_normed = false;
        }
        if (call.add_input) {
            if (x.dtype != DType::F32) throw ConfigError("adding the embedding's output back in needs a 32-bit residual stream");
            x = ops.add_scaled(x, x0, 1.0f);
            has_normed = false;
        }
        Norm* then = nullptr;
        if (i + 1 < n) then = layers[spec.program[i + 1].layer]->first_norm();
        else if (with_final_norm) then = final_norm.get();
        static const CacheView none;
        PartOut o = block->forward(ops, x, has_normed ? &normed : nullptr, with_values, call.cache >= 0 ? views[i] : none, then);
        x = o.x;
        if (dumping) dump_stream(ops, x, pass_no, i);
        has_normed = o.has_normed && then != nullptr;
        normed = o.normed;
    }
    ops.arena = outer;
    RunOut out;
    out.x = x;
    out.has_normed = has_normed && with_final_norm;
    out.normed = normed;
    return out;
}

Tensor DecoderModel::logits(Ops& ops, const Tensor& x, const int* rows, int64_t n_rows, const Rows* normed) {
    Rows h;
    if (rows) h = Rows(final_norm->forward(ops, ops.gather_rows(rows, n_rows, x)));
    else if (normed) h = *normed;
    else h = Rows(final_norm->forward(ops, x));
    Tensor out = ops.linear(h, head, nullptr, nullptr, (int)DType::F32);
    ops.finish_logits(out, head_bias.defined() ? &head_bias : nullptr, (float)spec.logit_scale, (float)spec.logit_softcap);
    return out;
}

}  // namespace friday
