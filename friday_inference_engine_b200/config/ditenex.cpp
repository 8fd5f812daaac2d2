// Ditenex: its config.json, checked and completed, and how it turns into parts.
//
// config.json is nested: "vocab", "width", "max_positions", "residual_mult", "norm": {"eps"}, and "layers": a list of
// {"type", "mixer", "mlp"}.  Every size and constant comes from there.
//
// The model: token rows plus the rows of a learned position table (32-bit stream); layers in order; final norm; the token
// table again as the head.  A layer is a block with an RMS norm before and after each sublayer and a multiplier m on what
// it adds, x <- x + m * norm_b(sublayer(norm(x))).  The mixer reads its input through a token shift (a blend with the row
// before, whose last one is part of a sequence's state).  The mixer is softmax attention behind a sliding window: grouped
// key/value heads, biased q/k/v projections, no rotation, a distance penalty 2^(-8 (h + 1) / heads) * (i - j) per head, the
// heads' scores mixed by a matrix before the softmax, values of a size of their own that layers with "v_mix" blend with the
// values of the first such layer, and a sigmoid gate on the heads' results.  The feed-forward is dense with a two-sided
// activation, or routed experts chosen by biased sigmoid scores among groups, with an expert that every token uses; or none.
#include "friday/config.h"
#include "friday/parts.h"

namespace friday {

namespace {
const char* kName = "Ditenex";
constexpr double kSlopeBase = 8.0;            // head h's distance penalty is 2^(-8 (h + 1) / heads) per position

const Json& member(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.is_object() ? d.find(key) : nullptr;
    if (!v || v->is_null()) throw ConfigError("config.json: " + where + " needs '" + key + "'");
    return *v;
}

int64_t positive_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_int() || v.as_int() <= 0) throw ConfigError("config.json: " + where + "'" + key + "' must be a positive integer");
    return v.as_int();
}

double number(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = member(d, key, where);
    if (!v.is_number()) throw ConfigError("config.json: " + where + "'" + key + "' must be a number");
    return v.as_double();
}

bool flag(const Json& d, const std::string& key) {
    const Json* v = d.is_object() ? d.find(key) : nullptr;
    return v && v->is_bool() && v->as_bool();
}

void check_attention(const Json& m, const std::string& where) {
    const int64_t heads = positive_int(m, "heads", where), kv = positive_int(m, "kv_heads", where);
    if (heads % kv) throw ConfigError(format("config.json: %s%lld heads cannot share %lld key/value heads", where.c_str(), (long long)heads, (long long)kv));
    positive_int(m, "dim", where);
    positive_int(m, "vdim", where);
    number(m, "scale", where);
    positive_int(member(m, "mask", where), "size", where + "mask: ");
}

void check_mlp(const Json& mlp, const std::string& where) {
    const std::string kind = member(mlp, "kind", where).as_string();
    if (kind == "dense") {
        positive_int(mlp, "ff", where);
        return;
    }
    if (kind != "moe") throw ConfigError("config.json: " + where + "feed-forward kind '" + kind + "' is not one this design has (dense, moe)");
    positive_int(member(mlp, "expert", where), "ff", where + "expert: ");
    const Json& router = member(mlp, "router", where);
    const std::string rw = where + "router: ";
    const int64_t experts = positive_int(router, "experts", rw), top = positive_int(router, "top", rw);
    number(router, "scale", rw);
    int64_t groups = 1, keep = 1;
    const Json* g = router.find("groups");
    if (g && !g->is_null()) {
        groups = positive_int(*g, "count", rw + "groups: ");
        keep = positive_int(*g, "keep", rw + "groups: ");
    }
    if (experts % groups || keep > groups || keep * (experts / groups) < top || top > experts)
        throw ConfigError(format("config.json: %s%lld experts in %lld groups of which %lld are kept cannot give %lld choices", rw.c_str(),
                                 (long long)experts, (long long)groups, (long long)keep, (long long)top));
    const Json* shared = mlp.find("shared");
    if (shared && !shared->is_null()) positive_int(*shared, "ff", where + "shared: ");
}

Json read_ditenex(const Json& d) {
    if (!d.is_object()) throw ConfigError("config.json: not an object");
    positive_int(d, "vocab", "");
    positive_int(d, "width", "");
    positive_int(d, "max_positions", "");
    number(d, "residual_mult", "");
    if (!(number(member(d, "norm", ""), "eps", "norm: ") > 0)) throw ConfigError("config.json: norm: 'eps' must be positive");
    const Json& layers = member(d, "layers", "");
    if (!layers.is_array() || layers.size() == 0) throw ConfigError("config.json: 'layers' must be a list of at least one layer");
    int64_t first_values = -1;                   // kv_heads * vdim of the first layer that blends values
    for (size_t i = 0; i < layers.size(); ++i) {
        const std::string where = format("layers[%zu]: ", i);
        const Json& type = member(layers[i], "type", where);
        if (type.as_string() != "attention")
            throw ConfigError("config.json: " + where + "mixer type '" + type.as_string() + "' is not one this design has (attention)");
        const Json& mixer = member(layers[i], "mixer", where);
        check_attention(mixer, where + "mixer: ");
        if (flag(mixer, "v_mix")) {
            // blended values are the first blending layer's, element by element: the rows must be as long
            const int64_t row = mixer.at("kv_heads").as_int() * mixer.at("vdim").as_int();
            if (first_values < 0) first_values = row;
            else if (row != first_values)
                throw ConfigError(format("config.json: %smixer: v_mix blends rows of kv_heads * vdim = %lld with the first such layer's %lld",
                                         where.c_str(), (long long)row, (long long)first_values));
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
    return PartSpec("rmsnorm", p, "");
}

// value_mix: "" (the layer does not blend), "first" or "blend"
PartSpec attention_spec(const Json& m, const std::string& value_mix) {
    Json p = Json::object();
    p.set("n_heads", m.at("heads"));
    p.set("n_kv_heads", m.at("kv_heads"));
    p.set("head_dim", m.at("dim"));
    p.set("v_head_dim", m.at("vdim"));
    p.set("scale", m.at("scale"));
    p.set("window", m.at("mask").at("size"));
    p.set("qkv_bias", Json(true));
    p.set("out_bias", Json(false));
    Json names = Json::object();
    for (const char* n : {"q", "k", "v", "o"}) names.set(n, Json(n));
    p.set("names", names);
    p.set("bias_suffix", Json(".b"));
    p.set("distance_slope_base", Json(kSlopeBase));
    p.set("talk", Json("talk"));
    p.set("gate", Json("g"));
    if (!value_mix.empty()) {
        p.set("value_mix", Json(value_mix));
        p.set("value_mix_weight", Json("vmix"));
    }
    PartSpec s("gqa_attention", p, "mix.");
    s.parts["position"] = PartSpec("none");
    return s;
}

PartSpec mlp_spec(const Json& mlp) {
    Json p = Json::object();
    if (mlp.at("kind").as_string() == "dense") {
        p.set("inner", mlp.at("ff"));
        p.set("activation", Json("two_sided"));
        return PartSpec("dense", p, "mlp.");
    }
    const Json& router = mlp.at("router");
    p.set("experts", router.at("experts"));
    p.set("top", router.at("top"));
    p.set("inner", mlp.at("expert").at("ff"));
    p.set("score", Json("sigmoid"));
    p.set("router_bias", Json(false));
    p.set("choice_bias", Json("correction"));
    p.set("weight_scale", router.at("scale"));
    const Json* g = router.find("groups");
    if (g && !g->is_null()) {
        p.set("groups", g->at("count"));
        p.set("groups_keep", g->at("keep"));
    }
    const Json* shared = mlp.find("shared");
    if (shared && !shared->is_null()) p.set("shared_inner", shared->at("ff"));
    return PartSpec("routed_experts", p, "mlp.");
}

ModelSpec ditenex_spec(const Json& c) {
    ModelSpec spec;
    spec.architecture = kName;
    spec.vocab_size = c.at("vocab").as_int();
    spec.width = c.at("width").as_int();
    spec.max_positions = c.at("max_positions").as_int();       // the position table has this many rows
    spec.embedding = "embed";
    spec.position_table = "pos";
    spec.residual_f32 = true;
    const double eps = c.at("norm").at("eps").as_double();
    spec.final_norm = norm_spec(eps, "final.norm");
    const Json& layers = c.at("layers");
    bool have_first = false;
    for (size_t i = 0; i < layers.size(); ++i) {
        const Json& L = layers[i];
        const std::string pre = format("l%zu.", i);
        Json bp = Json::object();
        bp.set("residual_mult", c.at("residual_mult"));
        bp.set("shift", Json("shift"));
        PartSpec block("sandwich", bp, pre);
        block.parts["norm1"] = norm_spec(eps, "norm1");
        block.parts["norm1b"] = norm_spec(eps, "norm1b");
        std::string value_mix;
        if (flag(L.at("mixer"), "v_mix")) {
            value_mix = have_first ? "blend" : "first";
            have_first = true;
        }
        if (value_mix != "blend") spec.ignorable.push_back(pre + "mix.vmix");       // the first blending layer's weight is not used
        block.parts["mixer"] = attention_spec(L.at("mixer"), value_mix);
        const Json* mlp = L.find("mlp");
        if (mlp && !mlp->is_null()) {
            block.parts["norm2"] = norm_spec(eps, "norm2");
            block.parts["norm2b"] = norm_spec(eps, "norm2b");
            block.parts["feed_forward"] = mlp_spec(*mlp);
        } else {
            spec.ignorable.push_back(pre + "norm2");          // a checkpoint may carry them all the same
            spec.ignorable.push_back(pre + "norm2b");
        }
        spec.layers.push_back(block);
        LayerCall call;
        call.layer = (int)i;
        call.cache = (int)i;
        spec.program.push_back(call);
    }
    return spec;
}

struct RegisterDitenex {
    RegisterDitenex() { register_architecture({kName, read_ditenex, ditenex_spec}); }
} register_ditenex;
}  // namespace

}  // namespace friday
