// Vulanex: its config.json, checked and completed, and how it turns into parts.
//
// config.json is nested: "vocab", "width", "logit_scale", "norm": {"eps"}, "canon": {"taps"}, "embedding": {"bigram":
// {"buckets", "mul_prev", "mul_cur"}}, "layers": a list of {"type", "mixer", "mlp"}.  Every size and constant comes from
// there (the inner size of the decay's two-step projection comes from the checkpoint's tensor shapes).
//
// The model: token rows plus the rows of a hashed table of token pairs, as a 32-bit residual stream; pre-norm layers with
// layer norms (weight and bias) whose sublayers read h + conv(h), a short causal convolution over time of the normed rows;
// a mixer that is either causal softmax attention without rotation whose values are its keys and whose queries grow with
// the position ("attention"), or two mixers side by side ("parallel": on the left attention with normed and rotated queries
// and keys behind a sliding window, with pooled blocks before the window and a sink per head, on the right the generalized
// delta rule), each result RMS-normed over the width, half their sum added to the stream; a gated feed-forward with the tanh
// form of gelu (or none); a final layer norm and the token table again as the head, times a multiplier.
#include "friday/config.h"
#include "friday/parts.h"

namespace friday {

namespace {
const char* kName = "Vulanex";

const Json& member(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.is_object() ? d.find(key) : nullptr;
    if (!v || v->is_null()) throw ConfigError("config.json: " + where + "needs '" + key + "'");
    return *v;
}

int64_t positive_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_int() || v.as_int() <= 0) throw ConfigError("config.json: " + where + "'" + key + "' must be a positive integer");
    return v.as_int();
}

int64_t natural_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_int() || v.as_int() < 0) throw ConfigError("config.json: " + where + "'" + key + "' must be an integer that is not negative");
    return v.as_int();
}

double number(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_number()) throw ConfigError("config.json: " + where + "'" + key + "' must be a number");
    return v.as_double();
}

void check_heads(const Json& m, const std::string& where) {
    const int64_t heads = positive_int(m, "heads", where), kv = positive_int(m, "kv_heads", where);
    if (heads % kv) throw ConfigError(format("config.json: %s%lld heads cannot share %lld key/value heads", where.c_str(), (long long)heads, (long long)kv));
    positive_int(m, "dim", where);
    positive_int(m, "vdim", where);
    number(m, "scale", where);
}

void check_attention(const Json& m, const std::string& where) {
    check_heads(m, where);
    if (m.at("dim").as_int() != m.at("vdim").as_int())
        throw ConfigError("config.json: " + where + "the values are the keys, so 'vdim' must equal 'dim'");
    const Json& qt = member(m, "q_temp", where);
    number(qt, "coef", where + "q_temp: ");
    positive_int(qt, "every", where + "q_temp: ");
}

void check_left(const Json& m, const std::string& where) {
    check_heads(m, where);
    const Json& mask = member(m, "mask", where);
    positive_int(mask, "size", where + "mask: ");
    positive_int(mask, "pool", where + "mask: ");
    const Json& rot = member(m, "rot", where);
    const std::string rw = where + "rot: ";
    if (!(number(rot, "base", rw) > 1.0)) throw ConfigError("config.json: " + rw + "'base' must be greater than 1");
    const int64_t dims = positive_int(rot, "dims", rw);
    if (dims > m.at("dim").as_int() || dims % 2) throw ConfigError("config.json: " + rw + "'dims' must be even and at most the mixer's 'dim'");
    const Json* sc = rot.find("scaling");
    if (sc && !sc->is_null())
        for (const char* k : {"factor", "original", "fast", "slow"})
            if (!(number(*sc, k, rw + "scaling: ") > 0)) throw ConfigError("config.json: " + rw + "scaling: '" + k + "' must be positive");
}

void check_right(const Json& m, const std::string& where) {
    positive_int(m, "heads", where);
    positive_int(m, "dim", where);
}

void check_mlp(const Json& mlp, const std::string& where) {
    const std::string kind = member(mlp, "kind", where).as_string();
    if (kind != "dense") throw ConfigError("config.json: " + where + "feed-forward kind '" + kind + "' is not one this design has (dense)");
    positive_int(mlp, "ff", where);
}

Json read_vulanex(const Json& d) {
    if (!d.is_object()) throw ConfigError("config.json: not an object");
    positive_int(d, "vocab", "");
    positive_int(d, "width", "");
    number(d, "logit_scale", "");
    if (!(number(member(d, "norm", ""), "eps", "norm: ") > 0)) throw ConfigError("config.json: norm: 'eps' must be positive");
    const int64_t taps = positive_int(member(d, "canon", ""), "taps", "canon: ");
    if (taps > 8) throw ConfigError("config.json: canon: 'taps' is at most 8");
    const Json& bg = member(member(d, "embedding", ""), "bigram", "embedding: ");
    positive_int(bg, "buckets", "embedding: bigram: ");
    natural_int(bg, "mul_prev", "embedding: bigram: ");
    natural_int(bg, "mul_cur", "embedding: bigram: ");
    const Json& layers = member(d, "layers", "");
    if (!layers.is_array() || layers.size() == 0) throw ConfigError("config.json: 'layers' must be a list of at least one layer");
    for (size_t i = 0; i < layers.size(); ++i) {
        const std::string where = format("layers[%zu]: ", i);
        const std::string type = member(layers[i], "type", where).as_string();
        const Json& mixer = member(layers[i], "mixer", where);
        if (type == "attention") {
            check_attention(mixer, where + "mixer: ");
        } else if (type == "parallel") {
            check_left(member(mixer, "left", where + "mixer: "), where + "mixer: left: ");
            check_right(member(mixer, "right", where + "mixer: "), where + "mixer: right: ");
        } else {
            throw ConfigError("config.json: " + where + "mixer type '" + type + "' is not one this design has (attention, parallel)");
        }
        const Json* mlp = layers[i].find("mlp");
        if (mlp && !mlp->is_null()) check_mlp(*mlp, where + "mlp: ");
    }
    Json v = d;                                   // complete as given; the names the registry looks for are added
    Json a = Json::array();
    a.push(Json(kName));
    v.set("architectures", a);
    v.set("architecture", Json(kName));
    return v;
}

PartSpec norm_spec(double eps, const std::string& tensor_name) {
    Json p = Json::object();
    p.set("eps", Json(eps));
    p.set("weight_name", Json(tensor_name));
    return PartSpec("layernorm", p, "");
}

// causal attention whose values are its keys, queries multiplied by a factor that grows with the position
PartSpec attention_spec(const Json& m, double eps, const std::string& prefix) {
    Json p = Json::object();
    for (const char* k : {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp"}) p.set(k, m.at(k));
    p.set("values", Json("keys"));
    p.set("eps", Json(eps));
    PartSpec s("pooled_attention", p, prefix);
    s.parts["position"] = PartSpec("none", Json::object(), "");
    return s;
}

// normed, rotated queries and keys behind a window, pooled blocks before it, a sink per head
PartSpec left_spec(const Json& m, double eps, const std::string& prefix) {
    Json p = Json::object();
    for (const char* k : {"heads", "kv_heads", "dim", "vdim", "scale"}) p.set(k, m.at(k));
    p.set("window", m.at("mask").at("size"));
    p.set("pool", m.at("mask").at("pool"));
    p.set("qk_norm", Json(true));
    p.set("sink", Json(true));
    p.set("eps", Json(eps));
    PartSpec s("pooled_attention", p, prefix);
    const Json& rot = m.at("rot");
    Json rp = Json::object();
    rp.set("base", rot.at("base"));
    rp.set("dims", rot.at("dims"));
    rp.set("layout", Json("halves"));
    const Json* sc = rot.find("scaling");
    if (sc && !sc->is_null()) rp.set("scaling", *sc);
    s.parts["position"] = PartSpec("rotary_pairs", rp, "");
    return s;
}

PartSpec right_spec(const Json& m, double eps, const std::string& prefix) {
    Json p = Json::object();
    p.set("heads", m.at("heads"));
    p.set("dim", m.at("dim"));
    p.set("eps", Json(eps));
    const Json* r = m.find("decay_rank");          // optional: for drawing random weights (a checkpoint's shapes give it)
    if (r && r->is_int() && r->as_int() > 0) p.set("decay_rank", *r);
    return PartSpec("general_delta", p, prefix);
}

ModelSpec vulanex_spec(const Json& c) {
    ModelSpec spec;
    spec.architecture = kName;
    spec.vocab_size = c.at("vocab").as_int();
    spec.width = c.at("width").as_int();
    spec.max_positions = (int64_t)1 << 30;            // nothing bounds a sequence but the cache
    spec.embedding = "embed";                         // also the head
    spec.residual_f32 = true;
    spec.logit_scale = c.at("logit_scale").as_double();
    const Json& bg = c.at("embedding").at("bigram");
    spec.pair_table.table = "bigram";
    spec.pair_table.buckets = bg.at("buckets").as_int();
    spec.pair_table.mul_prev = bg.at("mul_prev").as_int();
    spec.pair_table.mul_cur = bg.at("mul_cur").as_int();
    const double eps = c.at("norm").at("eps").as_double();
    spec.final_norm = norm_spec(eps, "final.norm");
    const Json& layers = c.at("layers");
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& L = layers[i];
        Json bp = Json::object(), conv = Json::object();
        conv.set("taps", c.at("canon").at("taps"));
        conv.set("mixer", Json("canon1"));
        conv.set("feed_forward", Json("canon2"));
        bp.set("input_conv", conv);
        PartSpec block("prenorm", bp, format("l%zu.", i));
        block.parts["norm1"] = norm_spec(eps, "norm1");
        const Json& m = L.at("mixer");
        if (L.at("type").as_string() == "attention") {
            block.parts["mixer"] = attention_spec(m, eps, "mix.");
        } else {
            Json pp = Json::object(), members = Json::array(), scales = Json::array(), norms = Json::array();
            members.push(Json("left"));
            members.push(Json("right"));
            scales.push(Json(0.5));
            scales.push(Json(0.5));
            norms.push(Json("left.out"));
            norms.push(Json("right.out"));
            pp.set("members", members);
            pp.set("scales", scales);
            pp.set("member_norms", norms);
            pp.set("eps", Json(eps));
            PartSpec par("parallel", pp, "mix.");
            par.parts["left"] = left_spec(m.at("left"), eps, "left.");
            par.parts["right"] = right_spec(m.at("right"), eps, "right.");
            block.parts["mixer"] = par;
        }
        const Json* mlp = L.find("mlp");
        if (mlp && !mlp->is_null()) {
            block.parts["norm2"] = norm_spec(eps, "norm2");
            Json p = Json::object();
            p.set("inner", mlp->at("ff"));
            p.set("activation", Json("gelu_tanh"));
            Json names = Json::object();
            for (const char* r : {"gate", "up", "down"}) names.set(r, Json(r));
            p.set("names", names);
            block.parts["feed_forward"] = PartSpec("swiglu", p, "mlp.");
        } else {
            for (const char* t : {"norm2", "norm2.b", "canon2"}) spec.ignorable.push_back(format("l%zu.%s", i, t));      // a checkpoint may carry them all the same
        }
        spec.layers.push_back(block);
        LayerCall call;
        call.layer = (int)i;
        call.cache = (int)i;
        spec.program.push_back(call);
    }
    return spec;
}

struct RegisterVulanex {
    RegisterVulanex() { register_architecture({kName, read_vulanex, vulanex_spec}); }
} register_vulanex;
}  // namespace

}  // namespace friday
